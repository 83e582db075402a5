"""Attention mixer over the paged cache."""

from __future__ import annotations

import numpy as np
import torch

from ..cache.manager import Retention
from ..kernels import api as K
from ..tracing import scope
from .base import KVNeed, LayerCache, Mixer, PositionEncoding, Runtime, StepContext, StepShape, register_part
from .linear import linear

# How this part's kernels cut a step's tokens (the planner below is theirs alone; nothing else knows these numbers).
FLASH_TILE = 16  # query rows per block of the mma.sync flash kernel
TC_TILE = 128  # query rows per block of the tcgen05 flash kernel
TC_MIN_TOKENS = 64  # a request that brings at least this many tokens goes to the tcgen05 kernel


def plan_attention_tiles(shape: StepShape) -> dict[str, np.ndarray]:
    """The step's tokens cut for the three attention kernels, once per step on the host.  A step of single
    tokens only needs no lists.  Otherwise, as int32 arrays of (first token row, count) pairs, each within one
    request: ``attn_tiles_all`` = every request that brings several tokens in tiles of FLASH_TILE;
    ``attn_tiles_long`` = requests that bring at least TC_MIN_TOKENS in tiles of TC_TILE; ``attn_tiles_short`` =
    the other requests with several tokens in tiles of FLASH_TILE; and ``attn_single_rows`` = the token rows of
    the requests that bring one token (decoded tokens beside the portions), which the split-KV kernel serves."""
    n_tok = np.asarray(shape.q_lens, dtype=np.int64)
    if n_tok.max() <= 1:
        return {}
    firsts = np.concatenate([[0], np.cumsum(n_tok)[:-1]])

    def cut(rows: int, which) -> np.ndarray:
        t = [(f + o, min(rows, n - o)) for f, n in zip(firsts, n_tok) if which(n) for o in range(0, n, rows)]
        # late tiles of a causal prompt read the most keys: launch them first so that the tail is short
        return np.ascontiguousarray(np.array(t, dtype=np.int32).reshape(-1, 2)[::-1])

    return {
        "attn_tiles_all": cut(FLASH_TILE, lambda n: n > 1),
        "attn_tiles_long": cut(TC_TILE, lambda n: n >= TC_MIN_TOKENS),
        "attn_tiles_short": cut(FLASH_TILE, lambda n: 1 < n < TC_MIN_TOKENS),
        "attn_single_rows": np.ascontiguousarray(firsts[n_tok == 1].astype(np.int32)),
    }


class PagedAttention(Mixer):
    """Grouped-query attention (llama4/llama4_jax/model.py:891-955, 745-794).

    ``w_qkv``: [(Hq + 2 Hkv) * dh, D], the q, k and v projections stacked in that order, each head a
    block of dh rows (HF orientation, chkpt_utils.py:84-89).  ``w_o``: [D, Hq * dh].
    ``chunk``: query and key must lie in the same chunk of that many positions (model.py:738-740);
    ``window``: keys within the last that many positions; None = no such limit.
    ``qk_norm_eps``: eps of the weightless norm of q and k, None = no norm.
    A layer with ``shares_cache`` projects only q and reads pages that another layer wrote.
    """

    kernel_libraries = ("attention_generic", "gemm_simt")
    kernel_libraries_bf16 = ("attention_mma", "attention_tc", "gemm_stream")

    def __init__(self, w_qkv: torch.Tensor, w_o: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: PositionEncoding, qk_norm_eps: float | None = None, chunk: int | None = None,
                 window: int | None = None, scale: float | None = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads are no multiple of {n_kv_heads} KV heads")
        rows = (n_heads + 2 * n_kv_heads) * head_dim
        if w_qkv.shape[0] != rows or w_o.shape[1] != n_heads * head_dim or w_o.shape[0] != w_qkv.shape[1]:
            raise ValueError(f"attention weights do not fit: w_qkv {tuple(w_qkv.shape)}, w_o {tuple(w_o.shape)} for "
                             f"{n_heads}/{n_kv_heads} heads of {head_dim}")
        self.w_qkv, self.w_o = w_qkv, w_o
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.position = position
        self.qk_norm_eps = qk_norm_eps
        self.chunk, self.window = chunk, window
        self.scale = float(head_dim) ** -0.5 if scale is None else float(scale)  # model.py:774

    # Head sizes that the tensor-core attention kernels are built for: a model with another head size never
    # asks for them (and so never compiles them).
    MMA_HEAD_SIZES = (64, 128)
    TC_HEAD_SIZES = (128,)

    def required_libraries(self, runtime: Runtime):
        return tuple(n for n in super().required_libraries(runtime)
                     if not (n == "attention_mma" and self.head_dim not in self.MMA_HEAD_SIZES)
                     and not (n == "attention_tc" and self.head_dim not in self.TC_HEAD_SIZES))

    def sub_parts(self):
        return (self.position,)

    def step_planners(self):
        return (plan_attention_tiles,)

    def kv_need(self) -> KVNeed:
        if self.chunk is not None and self.window is None:
            keep = Retention.chunk(self.chunk)
        elif self.window is not None and self.chunk is None:
            keep = Retention.window(self.window)
        else:
            keep = Retention.all()  # both limits at once: keep everything (correct, not minimal)
        return KVNeed(self.n_kv_heads, self.head_dim, keep)

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        rt = ctx.runtime
        with scope("qkv_matmul"):  # the scopes carry the reference's names (model.py:906-954)
            qkv = linear(ctx, h, self.w_qkv, rt.dtype, partials=self.position.accepts_partials)
        with scope("rope"):  # with the q/k norm and the cache update (the reference's "cache_update") in one kernel
            q = self.position.encode_and_store(ctx, qkv, self.n_heads, self.n_kv_heads, self.head_dim, cache, self.qk_norm_eps)
        attn_scale, floor_scale = self.position.query_temperature()
        out = torch.empty_like(q)
        with scope("attention"):
            self.attend(ctx, q, cache, out, attn_scale, floor_scale)
        with scope("projection"):
            return linear(ctx, out.view(q.shape[0], -1), self.w_o, torch.float32, partials=True)

    def _split_kv(self, ctx: StepContext, q, cache: LayerCache, out, attn_scale, floor_scale, rows, n_rows: int) -> None:
        """Split-KV attention for requests that bring one token: all rows of q, or the listed ones."""
        chunk, window = self.chunk or 0, self.window or 0
        split_keys, splits = K.attention_decode_plan(ctx.max_kv_len, chunk, window, n_rows * self.n_kv_heads)
        n = n_rows * self.n_heads * splits
        part_o = ctx.workspace.get("attn_part_o", n * self.head_dim, torch.float32)
        part_ml = ctx.workspace.get("attn_part_ml", n * 2, torch.float32)
        K.attention_decode(q, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, out, self.scale,
                           chunk, window, attn_scale, floor_scale, part_o, part_ml, splits, split_keys, ctx.status,
                           rows, n_rows)

    def attend(self, ctx: StepContext, q, cache: LayerCache, out, attn_scale: float, floor_scale: float) -> None:
        """Tensor-core kernels where they are built (bfloat16, head size 64 or 128, small groups): split-KV for
        requests that bring one token, flash tiles for the others (tcgen05 for long portions of head size 128);
        the generic kernel where those are not built."""
        chunk, window = self.chunk or 0, self.window or 0
        decode = ctx.max_q_len == 1
        if self.head_dim in self.MMA_HEAD_SIZES and K.attention_mma_supported(q.dtype, self.n_heads, self.n_kv_heads,
                                                                              self.head_dim, decode):
            if decode:
                self._split_kv(ctx, q, cache, out, attn_scale, floor_scale, None, q.shape[0])
                return
            tiles_all = ctx.arrays.get("attn_tiles_all")
            if tiles_all is not None:
                count = {name: len(a) for name, a in ctx.host_arrays.items()}
                if count["attn_single_rows"]:
                    # the single decoded tokens of a mixed step go to the split-KV kernel, by their row list
                    self._split_kv(ctx, q, cache, out, attn_scale, floor_scale, ctx.arrays["attn_single_rows"],
                                   count["attn_single_rows"])
                tiles, n_tiles = tiles_all, count["attn_tiles_all"]  # every request that brings more than one token
                if count["attn_tiles_long"] and self.head_dim in self.TC_HEAD_SIZES and K.attention_prefill_tc_supported(
                        q.dtype, self.n_heads, self.n_kv_heads, self.head_dim, cache.pages.shape[3]):
                    # long portions on the tcgen05 kernel (128-token tiles), the short ones below
                    K.attention_prefill_tc(q, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, out,
                                           ctx.arrays["attn_tiles_long"], count["attn_tiles_long"], self.scale, chunk, window,
                                           attn_scale, floor_scale, ctx.status)
                    tiles, n_tiles = ctx.arrays["attn_tiles_short"], count["attn_tiles_short"]
                    kinds = ("tc", "flash" if n_tiles else "", "split_kv" if count["attn_single_rows"] else "")
                    ctx.scratch.setdefault("attention_kernels", set()).add(tuple(k for k in kinds if k))
                if n_tiles:
                    K.attention_prefill(q, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, out, tiles,
                                        n_tiles, self.scale, chunk, window, attn_scale, floor_scale, ctx.status)
                return
        K.attention_generic(q, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, out, self.scale,
                            self.chunk or 0, self.window or 0, attn_scale, floor_scale, ctx.status)


register_part("mixer", "paged_attention", PagedAttention)
