"""The scheduler's decisions with the real host-side cache manager and a fake step function (no GPU)."""

import random

import pytest

from jax_llm_examples_b200.cache import CacheManager, Retention
from jax_llm_examples_b200.engine.scheduler import Request, Scheduler
from jax_llm_examples_b200.sampling import SamplingParams


def _setup(pages=16, page=16, slots=8, **kw):
    m = CacheManager(page, slots, 64)
    m.add_group(Retention.all(), pages)
    m.add_group(Retention.chunk(32), pages)
    batches = []

    def step_fn(entries):
        batches.append([(e.request.request_id, list(e.tokens), e.wants_logits) for e in entries])
        # the "model": next token = (sum of everything the request has in the cache after this step) % 97
        out = []
        for e in entries:
            if e.wants_logits:
                r = e.request
                out.append(sum(r.all_tokens[: r.fed + len(e.tokens)]) % 97)
        return out

    return m, Scheduler(m, step_fn, **kw), batches


def _expected(prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        out.append(sum(toks) % 97)
        toks.append(out[-1])
    return out


def test_prompt_is_cut_under_the_budget_and_only_its_end_asks_for_logits():
    m, s, batches = _setup(max_tokens_per_step=10)
    s.add(Request(0, list(range(1, 26)), SamplingParams(max_new_tokens=3)))
    s.run()
    assert [len(b[0][1]) for b in batches] == [10, 10, 5, 1, 1]
    assert [b[0][2] for b in batches] == [False, False, True, True, True]
    assert s.finished[0].output == _expected(range(1, 26), 3) and s.finished[0].finish_reason == "length"
    assert m.free_pages(0) == 16 and m.free_slots() == 8
    m.check()


def test_decodes_come_first_and_prompts_fill_the_rest():
    m, s, batches = _setup(max_tokens_per_step=8)
    s.add(Request(0, [1, 2, 3], SamplingParams(max_new_tokens=6)))
    s.step()
    s.add(Request(1, list(range(20)), SamplingParams(max_new_tokens=2)))
    s.step()
    rid_tokens = [(rid, len(t)) for rid, t, _ in batches[1]]
    assert rid_tokens == [(0, 1), (1, 7)]  # one decode token, then 7 of the budget for the new prompt
    s.run()
    outs = {r.request_id: r.output for r in s.finished}
    assert outs[0] == _expected([1, 2, 3], 6) and outs[1] == _expected(range(20), 2)
    assert all(sum(len(t) for _, t, _ in b) <= 8 for b in batches)


def test_admission_waits_for_slots_live_limit_and_pages():
    m, s, batches = _setup(pages=4, max_live=2)
    for i in range(3):
        s.add(Request(i, [5] * 20, SamplingParams(max_new_tokens=2)))
    s.step()
    assert [r.request_id for r in s.running] == [0, 1] and len(s.waiting) == 1  # 2 pages each: the pool is full
    s.run()
    assert sorted(r.request_id for r in s.finished) == [0, 1, 2]
    assert all(r.output == _expected([5] * 20, 2) for r in s.finished)
    m.check()


def test_eos_finishes_and_frees_at_once():
    m, s, _ = _setup()
    want = _expected([3, 4], 5)
    s.add(Request(0, [3, 4], SamplingParams(max_new_tokens=50, eos_token_ids=(want[2],))))
    s.run()
    assert s.finished[0].output == want[:3] and s.finished[0].finish_reason == "eos"
    assert m.free_pages(0) == 16


def test_running_out_of_pages_preempts_the_newest_and_recomputes_it():
    # 4 pages of 4 tokens: two requests of 6 prompt tokens grow until the pool is full
    m = CacheManager(4, 4, 16)
    m.add_group(Retention.all(), 4)
    seen = []

    def step_fn(entries):
        seen.append([(e.request.request_id, len(e.tokens)) for e in entries])
        return [sum(e.request.all_tokens[: e.request.fed + len(e.tokens)]) % 97 for e in entries if e.wants_logits]

    s = Scheduler(m, step_fn, max_tokens_per_step=64)
    a = Request(0, [1, 2, 3, 4, 5, 6], SamplingParams(max_new_tokens=9))
    b = Request(1, [9, 8, 7, 6, 5, 4], SamplingParams(max_new_tokens=4))
    s.add(a)
    s.add(b)
    s.run()
    assert a.output == _expected(a.prompt, 9) and b.output == _expected(b.prompt, 4)
    assert b.preemptions >= 1 and a.preemptions == 0  # the newest gives way, the oldest runs through
    assert any(p["preempted"] == [1] for p in s.log)
    # after the preemption request 1 came back with prompt + generated tokens as one portion
    assert any(rid == 1 and n > 6 for batch in seen for rid, n in batch)
    m.check()
    assert m.free_pages(0) == 4


def test_a_request_that_can_never_fit_is_finished_too_long():
    m, s, _ = _setup(pages=2)
    s.add(Request(0, [1] * 40, SamplingParams(max_new_tokens=2)))
    s.add(Request(1, [1] * 10, SamplingParams(max_new_tokens=2)))
    s.run()
    reasons = {r.request_id: r.finish_reason for r in s.finished}
    assert reasons == {0: "too_long", 1: "length"}
    m.check()


def test_prefills_that_block_each_other_are_resolved():
    m, s, _ = _setup(pages=5, max_tokens_per_step=24, max_portion=24)
    s.add(Request(0, [2] * 60, SamplingParams(max_new_tokens=2)))
    s.add(Request(1, [3] * 60, SamplingParams(max_new_tokens=2)))
    s.run()
    assert all(r.finish_reason == "length" for r in s.finished)
    assert {r.request_id: r.output for r in s.finished} == {0: _expected([2] * 60, 2), 1: _expected([3] * 60, 2)}
    m.check()


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_with_the_right_tokens(seed):
    rng = random.Random(seed)
    m, s, batches = _setup(pages=rng.choice([6, 12, 30]), page=rng.choice([4, 16]), slots=rng.choice([2, 4, 8]),
                           max_tokens_per_step=rng.choice([5, 16, 64]))
    reqs = []
    for i in range(12):
        prompt = [rng.randrange(50) for _ in range(rng.randrange(1, 40))]
        r = Request(i, prompt, SamplingParams(max_new_tokens=rng.randrange(1, 12)))
        reqs.append(r)
    pending = list(reqs)
    guard = 0
    while pending or s.has_work():
        if pending and rng.random() < 0.5:
            s.add(pending.pop(0))
        if s.has_work():
            s.step()
        m.check()
        guard += 1
        assert guard < 5000
    for r in reqs:
        if r.finish_reason == "too_long":
            pool = m.num_pages(0) * m.page_size
            assert len(r.prompt) + 1 > pool - m.page_size or len(r.all_tokens) + 1 > pool - m.page_size
            continue
        assert r.output == _expected(r.prompt, r.params.max_new_tokens), r.request_id
    assert all(m.free_pages(g) == m.num_pages(g) for g in range(2))
    assert all(sum(len(t) for _, t, _ in b) <= s.max_tokens_per_step for b in batches)
