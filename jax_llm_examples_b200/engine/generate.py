"""The Python entry point for generation: host token ids in, host token ids out.

The reference's offline path is ``prefill`` then a loop of ``decode_step`` over a fixed batch
(llama4/main.py:68-75, llama4/llama4_jax/model.py:1243-1277), greedy.  Here requests of any
lengths go through the scheduler and the one step function; tokens are sampled on the GPU and
only the chosen ids come back to the host each step.
"""

from __future__ import annotations

import time
from typing import Sequence

import torch

from ..parts.decoder import DecoderModel
from ..sampling.sampler import Sampler, SamplingParams, stream_of
from ..tracing import KernelTimer
from .engine import Engine, StepEntry
from .scheduler import PlannedEntry, Request, Scheduler


class Generator:
    """An engine, a scheduler and a sampler around one model."""

    def __init__(self, model: DecoderModel, *, max_tokens: int, page_size: int = 64, max_slots: int = 64,
                 max_tokens_per_step: int = 2048, max_live: int | None = None, max_seq_len: int | None = None,
                 seed: int = 0, profile: "bool | str" = False):
        self.engine = Engine(model, max_tokens=max_tokens, page_size=page_size, max_slots=max_slots,
                             max_seq_len=max_seq_len)
        self.sampler = Sampler(seed)
        self.scheduler = Scheduler(self.engine.manager, self._run, max_tokens_per_step=max_tokens_per_step,
                                   max_live=max_live, max_seq_len=self.engine.max_seq_len, on_admit=self._admit)
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._next_id = 0
        # profile=True: every step is timed on the host (the read of the sampled tokens ends it).
        # profile="kernels": also, every kernel launch is bracketed with CUDA events (no graph replay meanwhile);
        # ``kernel_timer.report()`` / ``.report("scope")`` give the times by kernel and by op group.
        self.profile = bool(profile)
        self.kernel_timer = KernelTimer() if profile == "kernels" else None
        self.step_times: list[tuple[int, int, float]] = []  # (prompt tokens, decode tokens, seconds)

    def _admit(self, r: Request) -> None:
        for s in self.engine.states:
            s[r.slot].zero_()

    def _run(self, entries: Sequence[PlannedEntry]) -> list[int]:
        batch = [StepEntry(e.request.slot, e.tokens, [len(e.tokens) - 1] if e.wants_logits else []) for e in entries]
        if self.profile:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
        try:
            if self.kernel_timer is not None:
                with self.kernel_timer:
                    return self._run_batch(entries, batch)
            return self._run_batch(entries, batch)
        finally:
            if self.profile:
                torch.cuda.synchronize()
                decode = sum(1 for e in entries if len(e.tokens) == 1 and e.request.output)
                self.step_times.append((sum(len(e.tokens) for e in entries) - decode, decode, time.perf_counter() - t0))

    def _run_batch(self, entries: Sequence[PlannedEntry], batch: list[StepEntry]) -> list[int]:
        logits = self.engine.step(batch)
        self.h2d_bytes += 4 * sum(len(e.tokens) for e in entries)
        want = [e.request for e in entries if e.wants_logits]
        if not want:
            return []
        toks = self.sampler.sample(
            logits, [r.params.temperature for r in want], [r.params.top_k for r in want],
            [stream_of(r.request_id, r.params) for r in want], [len(r.output) for r in want])
        host = toks.cpu()
        self.d2h_bytes += 4 * host.numel()
        self.engine.check_status()
        return host.tolist()

    def submit(self, prompt: Sequence[int], params: SamplingParams | None = None) -> Request:
        r = Request(self._next_id, list(prompt), params or SamplingParams())
        self._next_id += 1
        self.scheduler.add(r)
        return r

    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams] | None = None) -> list[list[int]]:
        """Generates for every prompt (token ids); returns the new token ids of each, in order."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        reqs = [self.submit(p, q) for p, q in zip(prompts, params)]
        self.scheduler.run()
        for r in reqs:
            if r.finish_reason == "too_long":
                raise ValueError(f"request {r.request_id} ({len(r.prompt)} prompt tokens) does not fit the cache "
                                 f"({self.engine.num_pages} pages of {self.engine.page_size} tokens)")
        return [r.output for r in reqs]


def generate(model: DecoderModel, prompts: Sequence[Sequence[int]], params: SamplingParams | None = None, *,
             page_size: int = 64, max_tokens: int | None = None, max_tokens_per_step: int = 2048, seed: int = 0) -> list[list[int]]:
    """One call: builds a Generator sized for these prompts and runs them."""
    params = params or SamplingParams()
    if max_tokens is None:
        max_tokens = sum(-(-(len(p) + params.max_new_tokens) // page_size) * page_size for p in prompts)
    gen = Generator(model, max_tokens=max_tokens, page_size=page_size, max_slots=max(len(prompts), 1),
                    max_tokens_per_step=max_tokens_per_step, seed=seed)
    return gen.generate(prompts, params)


# ------------------------------------------------------------------ the reference's two calls, on this engine
class Batch:
    """What ``prefill`` hands to ``decode_step``: an engine and one live request (cache slot) per prompt.  It
    stands where the reference passes its KVCache from call to call (llama4/llama4_jax/model.py:595-640)."""

    def __init__(self, engine: Engine, slots: list[int]):
        self.engine, self.slots = engine, slots
        self._scratch = (torch.empty(32 * len(slots), device=engine.runtime.device),
                         torch.empty(32 * len(slots), device=engine.runtime.device, dtype=torch.int32))

    def release(self) -> None:
        """Gives the requests' pages and slots back."""
        for s in self.slots:
            self.engine.finish(s)
        self.slots = []

    def _argmax(self, logits: torch.Tensor) -> torch.Tensor:
        from ..kernels import api as K

        out = torch.empty(logits.shape[0], device=logits.device, dtype=torch.int32)
        K.argmax(logits, out, *self._scratch)
        return out


def prefill(model_or_engine, prompts: Sequence[Sequence[int]], *, page_size: int = 64, max_new_tokens: int = 32):
    """The reference's ``prefill`` (llama4/llama4_jax/model.py:1243-1267): runs the prompts and returns
    (next token of each [B] on the host, logits at each prompt's last position [B, V] float32 on the device,
    the batch to decode on).  The reference pads the prompts to a common power of two and returns logits for
    every position; here each prompt runs at its own length and only the last position's logits are made.
    ``model_or_engine``: an Engine with room for the prompts, or a model, for which an engine is made that
    holds the prompts and ``max_new_tokens`` more tokens each."""
    if isinstance(model_or_engine, Engine):
        engine = model_or_engine
    else:
        need = sum(-(-(len(p) + max_new_tokens) // page_size) * page_size for p in prompts)
        engine = Engine(model_or_engine, max_tokens=need, page_size=page_size, max_slots=max(len(prompts), 1))
    slots = [engine.new_request() for _ in prompts]
    batch = Batch(engine, slots)
    logits = engine.step([StepEntry(s, list(p), [len(p) - 1]) for s, p in zip(slots, prompts)])
    next_tokens = batch._argmax(logits).cpu().tolist()
    engine.check_status()
    return next_tokens, logits, batch


def decode_step(batch: Batch, last_tokens: Sequence[int]):
    """The reference's ``decode_step`` (model.py:1270-1277): feeds each request its last token and returns
    (the next token of each by argmax, on the host; the batch)."""
    if len(last_tokens) != len(batch.slots):
        raise ValueError(f"{len(last_tokens)} tokens for {len(batch.slots)} requests")
    logits = batch.engine.step([StepEntry(s, [int(t)], [0]) for s, t in zip(batch.slots, last_tokens)])
    next_tokens = batch._argmax(logits).cpu().tolist()
    batch.engine.check_status()
    return next_tokens, batch
