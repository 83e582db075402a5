"""The step function: one batch of (request, its next tokens) through the model, from the cache.

The reference runs prompts and decoding as two separate programs over padded rectangular
batches (llama4/llama4_jax/model.py:1243-1277: ``prefill`` pads to a power of two, ``decode_step``
takes [B, 1]) on a ring-buffer cache.  Here one ``step`` takes any mixture: portions of prompts
of any length beside single decoded tokens, flattened to N token rows without padding.  It runs
only those tokens, reads everything earlier from the paged cache, writes their keys and values
into pages, and returns float32 logits at the places asked for.
"""

from __future__ import annotations

import dataclasses
import gc
from typing import Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, OutOfPages
from .. import tracing
from ..kernels import api as K
from ..parts.base import StepContext, StepShape, Workspace
from ..parts.decoder import DecoderModel


class EngineError(RuntimeError):
    pass


@dataclasses.dataclass
class StepEntry:
    """A request's share of a step: its next tokens and the places among them whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class _NotInAGraph:
    """Stands where a step's host copies would be while the step is captured in a CUDA graph."""

    def _refuse(self, *a, **k):
        raise EngineError("a part read the step's host copies (ctx.host_*) while the step was captured in a CUDA graph, "
                          "which would freeze this step's values into later steps: set `capturable = False` on that part")

    __iter__ = __len__ = __getitem__ = __bool__ = _refuse


class _HostRing:
    """Pinned host buffers for step descriptors; a buffer is reused only after its copy has run."""

    def __init__(self, n: int = 3):
        self.bufs: list[torch.Tensor | None] = [None] * n
        self.events: list[torch.cuda.Event | None] = [None] * n
        self.i = 0

    def next(self, size: int) -> tuple[torch.Tensor, int]:
        i = self.i
        self.i = (self.i + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        if self.bufs[i] is None or self.bufs[i].numel() < size:
            self.bufs[i] = torch.empty(max(size, 4096), dtype=torch.int32, pin_memory=True)
        return self.bufs[i], i

    def mark(self, i: int) -> None:
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class Engine:
    """Owns the cache (manager, pages, state slabs) of one model on one GPU and steps batches through it.

    ``max_tokens``: tokens that all live requests may hold together (each request's count rounded
    up to whole pages); every group's pool has ``ceil(max_tokens / page_size)`` pages.  None: as many
    as fit into ``memory_fraction`` of the GPU memory that is free when the engine is made.
    ``max_seq_len``: longest request (sets the block-table width); default ``max_tokens`` (131072 when the
    pool is sized from free memory).
    """

    DEFAULT_MAX_SEQ_LEN = 131072  # longest request when neither max_tokens nor max_seq_len says otherwise

    def __init__(self, model: DecoderModel, *, max_tokens: int | None, page_size: int = 64, max_slots: int = 64,
                 max_seq_len: int | None = None, use_graphs: bool | None = None, memory_fraction: float = 0.9):
        if not torch.cuda.is_available():
            raise EngineError("no CUDA device: this engine runs on a GPU only and has no CPU path")
        if max_tokens is None:
            max_tokens = self.tokens_that_fit(model, page_size, memory_fraction)
            if max_seq_len is None:  # a pool of millions of tokens: the block tables need not be that wide
                max_seq_len = min(max_tokens, self.DEFAULT_MAX_SEQ_LEN)
        if page_size <= 0 or max_tokens <= 0:
            raise EngineError("page_size and max_tokens must be positive")
        self.model, self.runtime = model, model.runtime
        self.page_size, self.max_slots = page_size, max_slots
        self.num_pages = -(-max_tokens // page_size)
        self.max_seq_len = max_seq_len or max_tokens
        self.max_pages_per_request = -(-self.max_seq_len // page_size)
        plan = model.plan
        K.preload(model.required_libraries())
        self.manager = CacheManager(page_size, max_slots, self.max_pages_per_request)
        for r in plan.groups:
            self.manager.add_group(r, self.num_pages)
        dev, dt = self.runtime.device, self.runtime.dtype
        self.kv = [torch.zeros((self.num_pages, 2, c.num_kv_heads, page_size, c.head_dim), dtype=dt, device=dev)
                   for c in plan.caches]
        self.states = [torch.zeros((max_slots, *s.shape), dtype=s.dtype, device=dev) for s in plan.states]
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._ring = _HostRing()
        self.workspace = Workspace(dev)
        self._dev_desc: torch.Tensor | None = None
        self.steps_run = 0
        self.record_routing = False  # True: keep each routed layer's expert choices of the last step
        self.last_routing: list[torch.Tensor] = []
        # Decode-only steps (one token per request) are launch-bound: from the second step of a batch
        # shape on, the step's kernels are captured once in a CUDA graph and replayed.  Per-request state lives
        # in static slabs indexed by the descriptor's slot ids, so a model with state is captured as well, unless
        # one of its parts says that it plans on the host (Part.capturable).
        self.use_graphs = (self.runtime.dtype == torch.bfloat16) if use_graphs is None else use_graphs
        self._graphs: dict[tuple[int, int, int], dict] = {}
        self._graph_pool = torch.cuda.graph_pool_handle() if self.use_graphs else None  # one pool for all graphs
        self._planners = model.step_planners()
        self._capturable = model.capturable
        self.last_scratch: dict = {}
        self.graph_replays = 0
        self.graph_kernel_launches = 0  # kernels of this package launched through graph replays

    @staticmethod
    def tokens_that_fit(model: DecoderModel, page_size: int = 64, memory_fraction: float = 0.9) -> int:
        """Tokens of cache (whole pages) that fit into this fraction of the device memory now free."""
        elem = 4 if model.runtime.dtype == torch.float32 else 2
        per_token = sum(2 * c.num_kv_heads * c.head_dim * elem for c in model.plan.caches)
        if per_token == 0:
            raise EngineError("this model keeps no keys and values: give max_tokens")
        free, _ = torch.cuda.mem_get_info(model.runtime.device)
        return int(free * memory_fraction / per_token) // page_size * page_size

    # ------------------------------------------------------------------ requests
    def new_request(self) -> int:
        """Takes a slot (raises OutOfSlots) and clears its per-request state."""
        slot = self.manager.alloc_slot()
        for s in self.states:
            s[slot].zero_()
        return slot

    def finish(self, slot: int) -> int:
        """Gives back everything the request holds; returns the number of pages given back."""
        return self.manager.release(slot)

    def length(self, slot: int) -> int:
        return self.manager.committed(slot)

    def cache_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv + self.states)

    # ---------------------------------------------------------------------- step
    def reserve(self, entries: Sequence[StepEntry]) -> None:
        """Takes the pages the entries need; raises OutOfPages (pages taken for earlier entries stay reserved)."""
        for e in entries:
            self.manager.reserve(e.slot, self.manager.committed(e.slot) + len(e.tokens))

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs one batch.  Returns float32 logits [M, vocab] on the device, M = all wanted places in
        the order of the entries and of each entry's ``want``.  The tensor may be a buffer that the next
        step overwrites (a replayed graph's): read or copy it before stepping again."""
        if not entries:
            raise EngineError("a step needs at least one entry")
        R = len(entries)
        n_tok = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=R)
        if (n_tok <= 0).any():
            raise EngineError("every entry of a step needs at least one token")
        if len({e.slot for e in entries}) != R:
            raise EngineError("a request may appear only once in a step")
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if tokens.min() < 0 or tokens.max() >= self.model.vocab_size:
            raise EngineError(f"token id outside the vocabulary [0, {self.model.vocab_size})")
        tokens = tokens.astype(np.int32)
        want_off = np.zeros(R + 1, dtype=np.int32)
        np.cumsum([len(e.want) for e in entries], out=want_off[1:])
        want = np.fromiter((w for e in entries for w in e.want), dtype=np.int32, count=int(want_off[-1]))
        slots = np.fromiter((e.slot for e in entries), dtype=np.int32, count=R)
        N, M = int(n_tok.sum()), int(want_off[-1])

        self.reserve(entries)
        starts = [self.manager.committed(e.slot) for e in entries]
        max_kv = max(s + int(n) for s, n in zip(starts, n_tok))
        G = len(self.manager.groups)
        # what the parts' planners make of this step (tile lists and the like); it travels with the descriptor
        shape = StepShape(tuple(int(n) for n in n_tok), tuple(starts), self.page_size, max_kv)
        extra: dict[str, np.ndarray] = {}
        for planner in self._planners:
            for name, a in planner(shape).items():
                extra[name] = np.ascontiguousarray(a, dtype=np.int32)
        extra_sizes = tuple((name, a.size) for name, a in extra.items())
        graph = None
        if self.use_graphs and N == R and not self.record_routing and self._capturable and not tracing.active():
            # A graph freezes the launch shapes, among them the split plan of decode attention, which is laid out
            # for a longest request: one graph per (requests, wanted rows, bucket of the longest request in the step).
            bucket = self.kv_bucket(max_kv)
            graph = self._graphs.setdefault((R, M, bucket), {"seen": 0, "extra": extra_sizes})
            graph["seen"] += 1
            if graph["extra"] != extra_sizes:
                graph = None  # a planner gave other sizes than the captured step had: run this step uncaptured
        static = graph is not None and graph["seen"] >= 2
        plan_kv = bucket if static else max_kv
        width = -(-plan_kv // self.page_size)
        packed = CacheManager.packed_size(G, N, R, M, width)
        size = packed + sum(a.size for a in extra.values())
        host, ring_i = self._ring.next(size)
        host_np = host.numpy()
        self.manager.pack_step(slots, n_tok, tokens, want_off, want, width, N, R, M, host_np)
        at = packed
        for a in extra.values():
            host_np[at:at + a.size] = a.reshape(-1)
            at += a.size
        if static:
            if "desc" not in graph:
                graph["desc"] = torch.empty(size, dtype=torch.int32, device=self.runtime.device)
            desc = graph["desc"]
        else:
            if self._dev_desc is None or self._dev_desc.numel() < size:
                self._dev_desc = torch.empty(max(size, 4096), dtype=torch.int32, device=self.runtime.device)
            desc = self._dev_desc[:size]
        desc.copy_(host[:size], non_blocking=True)
        self._ring.mark(ring_i)

        if static and "graph" in graph:
            graph["graph"].replay()
            self.graph_replays += 1
            self.graph_kernel_launches += graph["kernels"]
            logits = graph["logits"]
        else:
            o = 0

            def cut(n: int) -> torch.Tensor:
                nonlocal o
                v = desc[o:o + n]
                o += n
                return v

            # a captured step must not depend on this step's host copies: it is replayed for other steps
            host_view = (lambda v: _NotInAGraph()) if static else (lambda v: v)
            ctx = StepContext(
                runtime=self.runtime, n_tokens=N, n_requests=R,
                token_ids=cut(N), positions=cut(N), req_of_token=cut(N), cu_q=cut(R + 1), q_start=cut(R), kv_len=cut(R),
                slot_ids=cut(R), logit_rows=cut(M), n_logit_rows=M, status=self.status,
                host_q_lens=host_view([int(n) for n in n_tok]), host_q_start=host_view(starts),
                host_slot_ids=host_view([int(s) for s in slots]),
                max_q_len=int(n_tok.max()), max_kv_len=plan_kv, workspace=self.workspace,
            )
            block_tables = [cut(R * width).view(R, width) for _ in range(G)]
            for name, a in extra.items():
                ctx.host_arrays[name], ctx.arrays[name] = a, cut(a.size)
            if self.record_routing:
                ctx.scratch["record_routing"] = []
            if static:
                g = torch.cuda.CUDAGraph()
                # Graphs of engines that are no longer used die when Python collects them, and destroying a graph
                # is not allowed while another is being captured (it would spoil the capture): collect them now, and
                # capture in the mode that tolerates such calls from this thread.
                gc.collect()
                torch.cuda.synchronize()
                before = K.launch_count()
                with torch.cuda.graph(g, pool=self._graph_pool, capture_error_mode="relaxed"):
                    logits = self.model.forward(ctx, self.kv, self.states, block_tables)
                graph["graph"], graph["logits"], graph["kernels"] = g, logits, K.launch_count() - before
                g.replay()
                self.graph_replays += 1
                self.graph_kernel_launches += graph["kernels"]
            else:
                logits = self.model.forward(ctx, self.kv, self.states, block_tables)
            self.last_routing = ctx.scratch.get("record_routing", [])
            self.last_scratch = ctx.scratch
        for e, s, n in zip(entries, starts, n_tok):
            self.manager.commit(e.slot, s + int(n))
        self.steps_run += 1
        return logits

    KV_BUCKET_MIN = 1024  # below this many keys a decode step's attention is too short to be worth a plan of its own

    def kv_bucket(self, max_kv: int) -> int:
        """The longest-request length that a captured decode step is planned for: the step's own longest request
        rounded up to an eighth of its power of two (so a plan is at most an eighth too wide, and a request
        that grows from n to 2n tokens meets eight plans), within [KV_BUCKET_MIN, max_seq_len]."""
        b = self.KV_BUCKET_MIN
        if max_kv > b:
            step = (1 << (max_kv - 1).bit_length()) // 8
            b = -(-max_kv // step) * step
        return min(b, max(self.max_seq_len, 1))

    def check_status(self) -> None:
        """Reads the kernels' status word (synchronises) and raises if any kernel refused something."""
        bits = int(self.status.item())
        if bits:
            self.status.zero_()
            why = [text for bit, text in K.STATUS_BITS.items() if bits & bit]
            raise EngineError("a kernel reported: " + "; ".join(why))


__all__ = ["Engine", "EngineError", "OutOfPages", "StepEntry"]
