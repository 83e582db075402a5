"""Interfaces of the parts a decoder is put together from, and the step context they all see.

A part gets its sizes and constants as constructor arguments and never learns which model it
is in.  The kinds of part:

* :class:`Norm` — normalises rows of the residual stream.
* :class:`PositionEncoding` — turns projected q and k rows into position-aware ones and hands
  k and v to the cache.
* :class:`Mixer` — mixes information across a request's tokens (attention here); it says what it
  needs of the cache manager: pages of keys and values (:class:`KVNeed`) and/or per-request state
  of fixed size (:class:`StateNeed`).
* :class:`FeedForward` — acts on each token alone (dense, or routed experts).
* :class:`Block` — arranges the above (pre-norm residual block here).

All of them work on the *flattened* batch of a step: N token rows from R requests, described by
:class:`StepContext`.  The residual stream is float32 [N, D]; parts return a float32 ``delta`` that
the next norm adds to it (the sum is fused into the norm kernel).
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable

import torch

from ..cache.manager import Retention


@dataclasses.dataclass
class Runtime:
    """Where and in which precision a model runs."""

    dtype: torch.dtype  # activations and cache: torch.bfloat16, or torch.float32 for the true 32-bit path
    device: torch.device

    def __post_init__(self):
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be float32 or bfloat16, not {self.dtype}")


@dataclasses.dataclass(frozen=True)
class KVNeed:
    """Pages of keys and values: heads, head size, and which keys stay readable."""

    num_kv_heads: int
    head_dim: int
    retention: Retention


@dataclasses.dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size (zeroed when a request is admitted)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclasses.dataclass
class Rows:
    """Token rows that may still be split-K partials: ``data`` is [N, D], or float32 [splits, N, D] whose
    slices the consumer adds in ascending order (saving the launch that would add them).

    As a term of a :class:`RowSum` the rows may also lie elsewhere in ``data``: token r's row is ``base + r``, or,
    with ``index`` (int32 [N * k]), the sum of the k rows ``index[r * k + j]``, j ascending."""

    data: torch.Tensor
    splits: int = 1
    index: torch.Tensor | None = None
    k: int = 1
    base: int = 0


@dataclasses.dataclass
class RowSum:
    """A delta that is still a sum of terms, added in this order by a consumer that can (the RMSNorm kernel: it then
    does an expert layer's un-permute and sum, and no kernel runs for them alone).  ``materialize()`` makes the plain
    [N, D] float32 tensor for a consumer that cannot: :func:`as_rows` calls it."""

    terms: list[Rows]
    materialize: Callable[[], torch.Tensor]


def as_rows(x: "torch.Tensor | Rows | RowSum | None") -> "Rows | None":
    if x is None or isinstance(x, Rows):
        return x
    if isinstance(x, RowSum):
        return Rows(x.materialize(), 1)
    return Rows(x, 1)


class Workspace:
    """Named device buffers that live across steps (scratch of kernels, e.g. split-K partials).
    Kernels of one stream run in order, so a buffer can serve every layer in turn.  A buffer that was
    outgrown is kept, not freed: a captured CUDA graph may still hold its address."""

    def __init__(self, device: torch.device):
        self.device = device
        self._bufs: dict[str, torch.Tensor] = {}
        self._outgrown: list[torch.Tensor] = []
        self._side: torch.cuda.Stream | None = None

    def side_stream(self) -> torch.cuda.Stream:
        """A second stream for work that is independent of what the step's own stream does next (made on first use)."""
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        return self._side

    def zeros(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A buffer that is zero when first handed out and is never handed out as scratch: for kernels that keep a
        small state across launches (a ticket counter that every launch leaves at zero)."""
        key = "zeros:" + name
        t = self._bufs.get(key)
        if t is None or t.numel() < numel or t.dtype != dtype:
            if t is not None:
                self._outgrown.append(t)
            t = torch.zeros(max(numel, 1), dtype=dtype, device=self.device)
            self._bufs[key] = t
        return t[:numel]

    def get(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        t = self._bufs.get(name)
        if t is None or t.numel() < numel or t.dtype != dtype:
            if t is not None:
                self._outgrown.append(t)
            t = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._bufs[name] = t
        return t[:numel]


@dataclasses.dataclass
class LayerCache:
    """What one run of a layer sees of the cache in this step."""

    pages: torch.Tensor | None  # [num_pages, 2, Hkv, page_size, dh]
    block_table: torch.Tensor | None  # int32 [R, width], rows in the order of the step's requests
    writes: bool  # False: the layer reads a cache that another layer fills
    state: torch.Tensor | None  # [max_slots, *StateNeed.shape]


@dataclasses.dataclass
class StepContext:
    """One step's batch: N tokens of R requests, portions of prompts beside single decoded tokens."""

    runtime: Runtime
    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor  # int32 [N]
    positions: torch.Tensor  # int32 [N] absolute position in the request
    req_of_token: torch.Tensor  # int32 [N] index into this step's requests
    cu_q: torch.Tensor  # int32 [R + 1] token offsets of the requests
    q_start: torch.Tensor  # int32 [R] tokens the request held before this step
    kv_len: torch.Tensor  # int32 [R] tokens it holds after this step
    slot_ids: torch.Tensor  # int32 [R] cache-manager slot (indexes per-request state)
    logit_rows: torch.Tensor  # int32 [M] token rows whose logits are wanted
    n_logit_rows: int
    status: torch.Tensor  # int32 [1] error bits raised by kernels
    # host copies, for parts that plan on the host
    host_q_lens: list[int] = dataclasses.field(default_factory=list)
    host_q_start: list[int] = dataclasses.field(default_factory=list)
    host_slot_ids: list[int] = dataclasses.field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    scratch: dict[str, Any] = dataclasses.field(default_factory=dict)  # per-step memo shared by parts
    workspace: Workspace | None = None  # buffers that outlive the step
    # What the model's step planners (see :meth:`Part.step_planners`) made of this step, by name: int32 arrays
    # on the host, and the same arrays on the device (they travel with the step's descriptor, in its one copy).
    host_arrays: dict[str, Any] = dataclasses.field(default_factory=dict)
    arrays: dict[str, torch.Tensor] = dataclasses.field(default_factory=dict)

    def plan_with(self, planners, page_size: int) -> None:
        """Runs step planners for a context made by hand (a test of one part): what the engine does while it
        packs a step, with one small copy per array instead of the descriptor's single one."""
        shape = StepShape(tuple(self.host_q_lens), tuple(self.host_q_start), page_size, self.max_kv_len)
        for planner in planners:
            for name, a in planner(shape).items():
                self.host_arrays[name] = a
                self.arrays[name] = torch.tensor(a.tolist(), dtype=torch.int32).reshape(-1).to(self.token_ids.device)


@dataclasses.dataclass(frozen=True)
class StepShape:
    """What a step planner sees of a step, on the host, before anything runs."""

    q_lens: tuple[int, ...]  # tokens each request brings
    q_start: tuple[int, ...]  # tokens each request held before
    page_size: int
    max_kv_len: int


StepPlanner = Callable[["StepShape"], "dict[str, Any]"]


class Part:
    """Base of all parts.

    ``kernel_libraries``: the kernel libraries (``csrc/<name>.cu``) this part launches in every precision;
    ``kernel_libraries_bf16``: those it launches only with bfloat16 activations (tensor-core kernels: the
    32-bit path never builds or loads them).  Libraries are built on first use.
    """

    kernel_libraries: tuple[str, ...] = ()
    kernel_libraries_bf16: tuple[str, ...] = ()
    # False: forward() reads the step's host copies (``ctx.host_*``) or otherwise does work that a captured
    # CUDA graph would freeze; a model with such a part is never replayed from a graph.
    capturable: bool = True

    def required_libraries(self, runtime: Runtime) -> tuple[str, ...]:
        """What this part launches in this precision."""
        if runtime.dtype == torch.bfloat16:
            return tuple(dict.fromkeys(self.kernel_libraries + self.kernel_libraries_bf16))
        return self.kernel_libraries

    def step_planners(self) -> "tuple[StepPlanner, ...]":
        """Functions ``planner(shape: StepShape) -> {name: int32 numpy array}`` that this part wants run once per
        step on the host (tile lists, row lists and the like).  The model collects the distinct planners of all
        its parts; the engine runs each once per step and sends the arrays to the device together with the step's
        descriptor: ``ctx.arrays[name]`` (device) and ``ctx.host_arrays[name]``.  A planner is a module-level
        function (parts of the same kind share it, so it runs once however many layers use it) and must return
        the same names with the same sizes for steps of the same shape when it wants to be replayed from a graph."""
        return ()

    def sub_parts(self) -> "tuple[Part, ...]":
        """Parts inside this one (a block's norms, mixer and feed-forward; an attention's position encoding)."""
        return ()


def walk_parts(part: "Part"):
    yield part
    for p in part.sub_parts():
        yield from walk_parts(p)


@dataclasses.dataclass
class Dispatch:
    """What a routed feed-forward needs between the router and its experts' products: the step's (token, choice)
    pairs sorted by expert and the tokens' rows gathered (and scaled) in that order.  A feed-forward that can use
    them offers the buffers through ``router_request()``; a norm that routes for it may fill them in the same kernel
    and hands them back with the routing, which saves a decode step two dependent launches per layer."""

    counter: torch.Tensor  # int32 [1], zero between launches
    offsets: torch.Tensor  # int32 [groups + 1]
    sorted_pair: torch.Tensor  # int32 [pairs]
    sorted_pos: torch.Tensor  # int32 [pairs]
    tiles: "tuple[torch.Tensor, torch.Tensor] | None"  # (tile list, count) for the grouped streaming products
    a_sorted: torch.Tensor  # [pairs + extra_rows, D]
    extra_rows: int  # rows of a group appended after the experts (a shared expert that takes every token)
    tile_rows: int
    status: torch.Tensor


class Norm(Part):
    fuses_router: bool = False  # True: forward(router=...) also routes the tokens in its kernel

    def forward(self, ctx: StepContext, x: torch.Tensor, delta: "torch.Tensor | Rows | None", *, out_dtype: torch.dtype,
                want_f32: bool = False, row_index: torch.Tensor | None = None, router=None):
        """x += delta (if given); returns (normed rows in out_dtype, the same in float32 if asked,
        routing).  ``router`` = (w_router [E, D] float32, top_k) asks a norm with ``fuses_router`` to
        route as well: routing = (expert indices [N, k] int32, weights [N, k] float32); else None.  The request
        may have a third element, a function (ctx, n_rows) -> Dispatch or None; a norm that fills the Dispatch too
        returns it as the routing's third element."""
        raise NotImplementedError


class PositionEncoding(Part):
    accepts_partials: bool = False  # True: encode_and_store takes qkv as Rows with split-K partials

    def encode_and_store(self, ctx: StepContext, qkv: "torch.Tensor | Rows", n_heads: int, n_kv_heads: int, head_dim: int,
                         cache: LayerCache, qk_norm_eps: float | None) -> torch.Tensor:
        """qkv: [N, (Hq + 2 Hkv) * dh] projected rows.  Returns q [N, Hq, dh] ready for the score
        product; writes k and v into the cache pages when ``cache.writes``."""
        raise NotImplementedError

    def query_temperature(self) -> tuple[float, float]:
        """(attn_scale, floor_scale) of the position-dependent query scale; (0, 1) = none."""
        return (0.0, 1.0)


class Mixer(Part):
    def kv_need(self) -> KVNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache) -> "torch.Tensor | Rows":
        """h: normed rows [N, D] in the runtime's dtype.  Returns delta [N, D] float32 (or Rows of partials)."""
        raise NotImplementedError


class FeedForward(Part):
    needs_f32_input: bool = False  # True: forward() also gets the normed rows unrounded

    def router_request(self):
        """(w_router, top_k) if the preceding norm may route the tokens for this part, else None; optionally a third
        element, see Norm.forward."""
        return None

    def forward(self, ctx: StepContext, h: torch.Tensor, h32: torch.Tensor | None, routing=None) -> "torch.Tensor | Rows":
        """Returns delta [N, D] float32 (or Rows of partials).  ``routing``: what a fusing norm already chose."""
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, ctx: StepContext, x: torch.Tensor, delta: "torch.Tensor | Rows | None", cache: LayerCache):
        """Runs the block on residual x with a pending ``delta`` not yet added; returns the new pending delta."""
        raise NotImplementedError


# ------------------------------------------------------------------------------ part registry
_PARTS: dict[tuple[str, str], Callable[..., Part]] = {}
KINDS = ("norm", "position", "mixer", "feed_forward", "block")


def register_part(kind: str, name: str, factory: Callable[..., Part]) -> None:
    """Makes a part available to model builders under (kind, name)."""
    if kind not in KINDS:
        raise ValueError(f"unknown kind of part {kind!r}; kinds: {KINDS}")
    _PARTS[(kind, name)] = factory


def make_part(kind: str, name: str, **kwargs: Any) -> Part:
    try:
        factory = _PARTS[(kind, name)]
    except KeyError:
        known = sorted(n for k, n in _PARTS if k == kind)
        raise KeyError(f"no {kind} part named {name!r}; known: {known}") from None
    return factory(**kwargs)


def known_parts(kind: str) -> list[str]:
    return sorted(n for k, n in _PARTS if k == kind)
