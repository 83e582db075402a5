"""Feed-forward parts: dense SwiGLU and routed experts with a shared expert."""

from __future__ import annotations

import torch

from ..kernels import api as K
from ..tracing import active as tracing_active
from ..tracing import scope
from .base import Dispatch, FeedForward, Rows, RowSum, StepContext, as_rows, register_part
from .linear import (STREAM_MAX_ROWS, group_rows_hint, grouped_linear, grouped_swiglu_linear, grouped_swiglu_streams,
                     interleave_gate_up, linear,
                     swiglu_linear)


def _can_interleave(w_gate_up: torch.Tensor) -> bool:
    return w_gate_up.dtype == torch.bfloat16 and (w_gate_up.shape[-2] // 2) % 16 == 0 and w_gate_up.shape[-1] % 8 == 0


class DenseSwiGLU(FeedForward):
    """down(silu(h gate) * (h up)) (llama4/llama4_jax/model.py:1142-1153).
    ``w_gate_up``: [2F, D], gate rows then up rows; ``w_down``: [D, F].  bfloat16 weights are re-laid in
    blocks of [16 gate rows, 16 up rows] so that the product's epilogue can apply the activation."""

    kernel_libraries = ("elementwise", "gemm_simt")
    kernel_libraries_bf16 = ("gemm_stream",)

    def __init__(self, w_gate_up: torch.Tensor, w_down: torch.Tensor):
        if w_gate_up.shape[0] != 2 * w_down.shape[1] or w_gate_up.shape[1] != w_down.shape[0]:
            raise ValueError(f"SwiGLU weights do not fit: gate_up {tuple(w_gate_up.shape)}, down {tuple(w_down.shape)}")
        self.interleaved = _can_interleave(w_gate_up)
        self.w_gate_up = interleave_gate_up(w_gate_up) if self.interleaved else w_gate_up
        self.w_down = w_down

    def forward(self, ctx: StepContext, h, h32=None, routing=None):
        with scope("gate_up_proj"):  # the reference's "gate" and "up_proj" (model.py:1145-1149) as one product
            act = swiglu_linear(ctx, h, self.w_gate_up, self.interleaved, ctx.runtime.dtype)
        with scope("down_proj"):
            return linear(ctx, act, self.w_down, torch.float32, partials=True)


class RoutedExperts(FeedForward):
    """Sigmoid-routed top-k experts plus an optional shared expert (model.py:958-972, 999-1139).

    scores = h W_router in float32 from the unrounded normed rows; top-k of the raw scores (lower
    index wins ties); weight = sigmoid(score); each chosen expert runs SwiGLU on weight * h (the
    INPUT is scaled, model.py:1071); expert outputs are summed per token in choice order and the
    shared expert's output on the unscaled h is added (model.py:1111, 1137-1139).
    ``w_router``: [E, D]; ``we_gate_up``: [E, 2F, D] (gate rows then up rows); ``we_down``: [E, D, F]."""

    kernel_libraries = ("moe", "elementwise", "gemm_simt")
    kernel_libraries_bf16 = ("gemm_stream",)
    needs_f32_input = True
    OVERLAP_MIN_ROWS = 512  # from this many rows on (prompt portions), the shared expert runs on a second stream beside the routed ones
    FORK_MIN_ROWS = 2  # and in steps of few rows (decoding) from this many on; below, it rides as a group of the routed products

    def __init__(self, w_router: torch.Tensor, we_gate_up: torch.Tensor, we_down: torch.Tensor, top_k: int,
                 shared: DenseSwiGLU | None = None):
        E = w_router.shape[0]
        if we_gate_up.shape[0] != E or we_down.shape[0] != E or we_gate_up.shape[1] != 2 * we_down.shape[2] \
                or we_gate_up.shape[2] != we_down.shape[1] or w_router.shape[1] != we_down.shape[1]:
            raise ValueError(f"expert weights do not fit: router {tuple(w_router.shape)}, gate_up "
                             f"{tuple(we_gate_up.shape)}, down {tuple(we_down.shape)}")
        if not 1 <= top_k <= E:
            raise ValueError(f"top-{top_k} of {E} experts")
        self.w_router = w_router.to(torch.float32).contiguous()
        self.interleaved = _can_interleave(we_gate_up)
        self.we_gate_up = interleave_gate_up(we_gate_up) if self.interleaved else we_gate_up
        self.we_down, self.top_k, self.shared = we_down, top_k, shared
        self.num_experts = E
        # A shared expert of the experts' own shape rides along as group E of the grouped products when a step
        # has few rows (decoding): two launches fewer, and its weights stream at the grouped kernel's rate.
        # Its weights then live at the end of the experts' tensors; the shared part keeps views of them.
        self.merged = (shared is not None and shared.interleaved == self.interleaved
                       and shared.w_gate_up.shape == self.we_gate_up.shape[1:] and shared.w_down.shape == we_down.shape[1:]
                       and shared.w_gate_up.dtype == self.we_gate_up.dtype == torch.bfloat16 and shared.w_down.dtype == we_down.dtype)
        if self.merged:
            self.we_gate_up = torch.cat([self.we_gate_up, shared.w_gate_up[None]])
            self.we_down = torch.cat([self.we_down, shared.w_down[None]])
            shared.w_gate_up, shared.w_down = self.we_gate_up[E], self.we_down[E]

    def sub_parts(self):
        return () if self.shared is None else (self.shared,)

    def router_request(self):
        return (self.w_router, self.top_k, self.offer_dispatch)

    def placement(self, ctx: StepContext, n: int) -> tuple[bool, bool]:
        """Where the shared expert runs in a step of n rows: (on a second stream beside the routed experts, as one more
        group of the routed experts' products).  One row: as a group (two launches fewer; with so few blocks one
        kernel streams better than two).  More rows: on a second stream, beside the routed products: its weights stream
        while the routed products' few blocks leave memory bandwidth unused, or their short predecessors leave it idle
        (decode at batch 2: +7.5 %, batch 8: +3.7 %, batch 64: +6.5 %; batch 1 would lose 2 %).  Prompt portions: the routed experts stream their weights once for
        about a hundred rows each (bound by HBM), the shared expert's products are dense (bound by the tensor cores);
        side by side, the tails and the small kernels of either hide behind the other.  Between STREAM_MAX_ROWS and
        OVERLAP_MIN_ROWS: one after the other."""
        beside = self.shared is not None and ctx.workspace is not None and (
            self.FORK_MIN_ROWS <= n <= STREAM_MAX_ROWS or n >= self.OVERLAP_MIN_ROWS)
        return beside, self.merged and n <= STREAM_MAX_ROWS and not beside

    def sort_buffers(self, ctx: StepContext, n: int, extra_rows: int):
        """(offsets, sorted_pair, sorted_pos, tiles, tile_rows) for a step of n rows, not yet filled."""
        k, dev = self.top_k, self.w_router.device
        offsets = torch.empty(self.num_experts + 2, dtype=torch.int32, device=dev)
        sorted_pair = torch.empty(n * k, dtype=torch.int32, device=dev)
        sorted_pos = torch.empty(n * k, dtype=torch.int32, device=dev)
        tiles, tile_rows = None, 0
        if self.we_gate_up.dtype == torch.bfloat16 and ctx.runtime.dtype == torch.bfloat16:
            # the grouped products will run on the streaming kernel: their row tiles are listed once, by the sort
            rows, groups = n * k + extra_rows, self.num_experts + (extra_rows > 0)
            tile_rows = K.gemm_stream_token_tile(group_rows_hint(rows, groups, extra_rows))
            tiles = (torch.empty(2 * (-(-rows // tile_rows) + groups), dtype=torch.int32, device=dev),
                     torch.empty(1, dtype=torch.int32, device=dev))
        return offsets, sorted_pair, sorted_pos, tiles, tile_rows

    def offer_dispatch(self, ctx: StepContext, n: int) -> Dispatch | None:
        """The buffers that a norm which routes for this part may fill as well (see Dispatch)."""
        if ctx.workspace is None:
            return None
        extra = n if self.placement(ctx, n)[1] else 0
        offsets, sorted_pair, sorted_pos, tiles, tile_rows = self.sort_buffers(ctx, n, extra)
        a_sorted = torch.empty((n * self.top_k + extra, self.w_router.shape[1]), dtype=ctx.runtime.dtype, device=self.w_router.device)
        return Dispatch(ctx.workspace.zeros("dispatch_counter", 1, torch.int32), offsets, sorted_pair, sorted_pos, tiles, a_sorted,
                        extra, tile_rows, ctx.status)

    def route(self, ctx: StepContext, h32: torch.Tensor):
        """The router as a kernel of its own (when the norm before this part does not route)."""
        n, k, dev = h32.shape[0], self.top_k, h32.device
        topk_idx = torch.empty((n, k), dtype=torch.int32, device=dev)
        topk_w = torch.empty((n, k), dtype=torch.float32, device=dev)
        K.router(h32, self.w_router, topk_idx, topk_w)
        return topk_idx, topk_w

    def sort(self, ctx: StepContext, topk_idx: torch.Tensor, extra_rows: int = 0):
        offsets, sorted_pair, sorted_pos, tiles, tile_rows = self.sort_buffers(ctx, topk_idx.shape[0], extra_rows)
        if tiles is not None:
            K.expert_sort(topk_idx, offsets, sorted_pair, sorted_pos, self.num_experts, ctx.status, extra_rows, tile_rows, *tiles)
        else:
            K.expert_sort(topk_idx, offsets, sorted_pair, sorted_pos, self.num_experts, ctx.status, extra_rows)
        return offsets, sorted_pair, sorted_pos, tiles

    def forward(self, ctx: StepContext, h, h32, routing=None):
        rt = ctx.runtime
        n, D = h32.shape
        k, E = self.top_k, self.num_experts
        topk_idx, topk_w, *dispatched = routing if routing is not None else self.route(ctx, h32)
        done = dispatched[0] if dispatched else None  # sorted and gathered already, by the norm that routed
        if "record_routing" in ctx.scratch:  # tests compare the choices with a plain router's
            ctx.scratch["record_routing"].append(topk_idx)
        beside, merged = self.placement(ctx, n)
        extra = n if merged else 0
        shared, side = None, None
        if beside:
            main, side = torch.cuda.current_stream(), ctx.workspace.side_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side), scope("moe_shared_expert"):
                shared = as_rows(self.shared.forward(ctx, h, None))
            shared.data.record_stream(main)  # made on the side stream, read (and freed) on the step's own
        with scope("moe_routed_expert"):  # the reference's names (model.py:1076-1138)
            if done is not None:
                if done.extra_rows != extra:
                    raise RuntimeError("the rows gathered with the routing do not fit this step's placement of the shared expert")
                offsets, sorted_pos, tiles, a_sorted = done.offsets, done.sorted_pos, done.tiles, done.a_sorted
            else:
                with scope("permute"):
                    offsets, sorted_pair, sorted_pos, tiles = self.sort(ctx, topk_idx, extra)
                    a_sorted = torch.empty((n * k + extra, D), dtype=rt.dtype, device=h.device)
                    K.permute_scale(h32, sorted_pair, topk_w, a_sorted, k, extra)
            groups = E + 1 if merged else E
            with scope("we_gate_up"):
                one_product = grouped_swiglu_streams(a_sorted, self.we_gate_up[:groups], self.interleaved)
                act = grouped_swiglu_linear(ctx, a_sorted, self.we_gate_up[:groups], offsets, self.interleaved, rt.dtype, extra, tiles)
            with scope("we_down"):  # (a timer's events between the two launches would come between them on the stream)
                y = grouped_linear(ctx, act, self.we_down[:groups], offsets, torch.float32, partials=True, largest_group=extra,
                                   tiles=tiles, after_grouped=one_product and not tracing_active())
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        elif self.shared is not None and not merged:
            with scope("moe_shared_expert"):
                shared = as_rows(self.shared.forward(ctx, h, None))
        def combine() -> torch.Tensor:
            delta = torch.empty((n, D), dtype=torch.float32, device=h.device)
            with scope("unpermute"):  # with the reference's "expert_summing" in the same kernel
                K.moe_combine(y.data, None if shared is None else shared.data, sorted_pos, delta, k,
                              1 if shared is None else shared.splits, y.splits, n * k if merged else -1)
            return delta

        # The un-permute and the sum over a token's experts are left to the consumer (the next norm adds the rows
        # where it adds the residual); the order is the combine kernel's: shared expert, then the experts by choice.
        if y.data.dtype != torch.float32 or (shared is not None and shared.data.dtype != torch.float32):
            return combine()
        terms = [shared] if shared is not None else []
        if merged:
            terms.append(Rows(y.data, y.splits, None, 1, n * k))
        terms.append(Rows(y.data, y.splits, sorted_pos, k, 0))
        return RowSum(terms, combine)


register_part("feed_forward", "dense_swiglu", DenseSwiGLU)
register_part("feed_forward", "routed_experts", RoutedExperts)
