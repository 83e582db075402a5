"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

The reference's offline driver prefills a fixed batch whole and decodes 32 steps
(llama4/main.py:68-74).  Its serving loop (serving/serving_jax/serving_loop.py) admits from a FIFO
queue while a decode slot is free (:613-625), prefills whole prompts padded to a power of two
(:699-708) and finishes on EOS or a length limit (:650-660); it has no token budget and no answer
to a full cache.  The policy here, each step:

1. Every running request that has a sampled token to feed gets one decode token.  If the pools
   cannot give the page it needs, the most recently admitted running request is *preempted*: all
   its pages and its slot are given back and it returns to the FRONT of the waiting queue with
   prompt + tokens generated so far, to be recomputed later.  (Random draws are keyed by the
   request's own step count, so the recomputed request continues with the same tokens.)
2. What is left of ``max_tokens_per_step`` goes to prompts: first requests whose prompt is partly
   in the cache, then waiting ones in arrival order, admitted while a slot is free, fewer than
   ``max_live`` are live and pages for the portion are free.  A portion is at most ``max_portion``
   tokens and may be cut anywhere; only the portion that ends the prompt asks for logits.
   Prompts never preempt anything: they wait.
3. A request that cannot run even with every page free is finished with reason ``"too_long"``.

The scheduler owns no GPU code: ``step_fn(entries) -> tokens`` runs the batch and samples; the
cache manager is the host-side one, so every decision can be tested without a GPU.
"""

from __future__ import annotations

import collections
import dataclasses
from typing import Callable, Sequence

from ..cache.manager import CacheManager, OutOfPages
from ..sampling.sampler import SamplingParams


@dataclasses.dataclass
class Request:
    request_id: int
    prompt: list[int]
    params: SamplingParams = dataclasses.field(default_factory=SamplingParams)
    # filled by the scheduler
    output: list[int] = dataclasses.field(default_factory=list)
    slot: int | None = None
    fed: int = 0  # tokens of (prompt + output) that are in the cache
    finish_reason: str | None = None
    preemptions: int = 0
    admitted_at: int = -1

    @property
    def all_tokens(self) -> list[int]:
        return self.prompt + self.output

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None


@dataclasses.dataclass
class PlannedEntry:
    request: Request
    tokens: list[int]
    wants_logits: bool  # the entry's last token yields the request's next token


StepFn = Callable[[Sequence[PlannedEntry]], Sequence[int]]
"""Runs the entries as one batch; returns one sampled token per entry with wants_logits, in order."""


class Scheduler:
    def __init__(self, manager: CacheManager, step_fn: StepFn, *, max_tokens_per_step: int = 2048,
                 max_live: int | None = None, max_portion: int | None = None, max_seq_len: int | None = None,
                 on_admit: Callable[[Request], None] | None = None):
        if max_tokens_per_step < 1:
            raise ValueError("max_tokens_per_step must be >= 1")
        self.manager, self.step_fn = manager, step_fn
        self.max_tokens_per_step = max_tokens_per_step
        self.max_live = max_live if max_live is not None else manager.max_slots
        self.max_portion = max_portion or max_tokens_per_step
        self.max_seq_len = max_seq_len or manager.max_pages_per_request * manager.page_size
        self.on_admit = on_admit
        self.waiting: collections.deque[Request] = collections.deque()
        self.running: list[Request] = []  # in admission order
        self.finished: list[Request] = []
        self.step_count = 0
        self._admissions = 0
        self.log: list[dict] = []  # one record per step: what was decided

    # ------------------------------------------------------------------ intake
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---------------------------------------------------------------- planning
    def _finish(self, r: Request, reason: str) -> None:
        r.finish_reason = reason
        if r.slot is not None:
            self.manager.release(r.slot)
            r.slot = None
        if r in self.running:
            self.running.remove(r)
        self.finished.append(r)

    def _preempt(self, r: Request) -> None:
        self.manager.release(r.slot)
        r.slot, r.fed = None, 0
        r.preemptions += 1
        self.running.remove(r)
        self.waiting.appendleft(r)

    def _fits_empty_pool(self, n_tokens: int) -> bool:
        pages = -(-n_tokens // self.manager.page_size)
        return (pages <= min(self.manager.num_pages(g) for g in range(len(self.manager.groups)))
                and pages <= self.manager.max_pages_per_request)

    def plan(self) -> tuple[list[PlannedEntry], list[Request]]:
        """Decides the next step.  Returns (entries, requests preempted while planning)."""
        budget = self.max_tokens_per_step
        entries: list[PlannedEntry] = []
        preempted: list[Request] = []

        # 1. decode tokens: running requests with exactly one token left to feed
        for r in list(self.running):
            if r not in self.running or budget == 0:
                continue
            if not r.output or r.fed != len(r.prompt) + len(r.output) - 1:
                continue  # still has a prompt (or a recomputation) to feed: handled below
            while True:
                try:
                    self.manager.reserve(r.slot, r.fed + 1)
                    entries.append(PlannedEntry(r, [r.output[-1]], True))
                    budget -= 1
                    break
                except OutOfPages:
                    victim = self.running[-1]
                    for e in [e for e in entries if e.request is victim]:
                        entries.remove(e)
                        budget += len(e.tokens)
                    self._preempt(victim)
                    preempted.append(victim)
                    if victim is r:
                        break

        # 2. prompt portions: partly cached prompts first, then the waiting queue.  A preempted
        # request's "prompt" is everything it had: its prompt and the tokens it generated.
        def portion(r: Request) -> bool:
            nonlocal budget
            seq = r.all_tokens
            n = min(len(seq) - r.fed, budget, self.max_portion)
            if n <= 0:
                return False
            try:
                self.manager.reserve(r.slot, r.fed + n)
            except OutOfPages:
                return False
            entries.append(PlannedEntry(r, seq[r.fed:r.fed + n], r.fed + n == len(seq)))
            budget -= n
            return True

        for r in self.running:
            if budget == 0:
                break
            if any(e.request is r for e in entries):
                continue
            portion(r)

        while self.waiting and budget > 0 and len(self.running) < self.max_live and self.manager.free_slots() > 0:
            r = self.waiting[0]
            if r in preempted:
                break  # give its pages a step to be used by the others
            if not self._fits_empty_pool(len(r.all_tokens) + 1) or len(r.all_tokens) >= self.max_seq_len:
                self.waiting.popleft()
                self._finish(r, "too_long")
                continue
            first = min(len(r.all_tokens), budget, self.max_portion)
            probe_pages = -(-first // self.manager.page_size)
            if any(self.manager.free_pages(g) < probe_pages for g in range(len(self.manager.groups))):
                break
            self.waiting.popleft()
            r.slot = self.manager.alloc_slot()
            r.fed = 0
            r.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(r)
            if self.on_admit:
                self.on_admit(r)
            if not portion(r):
                break
        return entries, preempted

    # ----------------------------------------------------------------- running
    def step(self) -> list[Request]:
        """Plans and runs one step; returns the requests that finished in it."""
        done_before = len(self.finished)
        entries, preempted = self.plan()
        while not entries and self.running:
            # every live request waits for pages that the others hold: the newest one gives way
            victim = self.running[-1]
            self._preempt(victim)
            preempted.append(victim)
            more, pre2 = self.plan()
            entries, preempted = more, preempted + pre2
            if not self.running and not entries:
                break
        if not entries:
            if self.waiting and not self.running:
                # nothing is live and the head of the queue still cannot start: it can never run
                r = self.waiting.popleft()
                self._finish(r, "too_long")
            return self.finished[done_before:]
        sampled = list(self.step_fn(entries))
        self.log.append({"step": self.step_count, "tokens": sum(len(e.tokens) for e in entries),
                         "decode": sum(1 for e in entries if len(e.tokens) == 1 and e.request.output),
                         "portions": [(e.request.request_id, len(e.tokens)) for e in entries if not (len(e.tokens) == 1 and e.request.output)],
                         "preempted": [r.request_id for r in preempted]})
        self.step_count += 1
        it = iter(sampled)
        for e in entries:
            r = e.request
            r.fed += len(e.tokens)
            self.manager.commit(r.slot, r.fed)
            if not e.wants_logits:
                continue
            tok = int(next(it))
            r.output.append(tok)
            if tok in r.params.eos_token_ids:
                self._finish(r, "eos")
            elif len(r.output) >= r.params.max_new_tokens:
                self._finish(r, "length")
            elif len(r.prompt) + len(r.output) >= self.max_seq_len:
                self._finish(r, "context")
        return self.finished[done_before:]

    def run(self) -> list[Request]:
        while self.has_work():
            self.step()
        return self.finished
