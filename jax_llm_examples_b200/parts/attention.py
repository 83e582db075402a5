"""Attention mixer over the paged cache."""

from __future__ import annotations

import torch

from ..cache.manager import Retention
from ..kernels import api as K
from .base import KVNeed, LayerCache, Mixer, PositionEncoding, Runtime, StepContext, register_part
from .linear import linear


class PagedAttention(Mixer):
    """Grouped-query attention (llama4/llama4_jax/model.py:891-955, 745-794).

    ``w_qkv``: [(Hq + 2 Hkv) * dh, D], the q, k and v projections stacked in that order, each head a
    block of dh rows (HF orientation, chkpt_utils.py:84-89).  ``w_o``: [D, Hq * dh].
    ``chunk``: query and key must lie in the same chunk of that many positions (model.py:738-740);
    ``window``: keys within the last that many positions; None = no such limit.
    ``qk_norm_eps``: eps of the weightless norm of q and k, None = no norm.
    A layer with ``shares_cache`` projects only q and reads pages that another layer wrote.
    """

    kernel_libraries = ("attention_generic", "attention_mma", "attention_tc", "rope_kv", "gemm_simt", "gemm_stream")

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
        mine = [n for n in super().required_libraries(runtime)
                if not (n == "attention_mma" and self.head_dim not in self.MMA_HEAD_SIZES)
                and not (n == "attention_tc" and self.head_dim not in self.TC_HEAD_SIZES)]
        return tuple(dict.fromkeys(tuple(mine) + self.position.required_libraries(runtime)))

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
        qkv = linear(ctx, h, self.w_qkv, rt.dtype, partials=self.position.accepts_partials)
        q = self.position.encode_and_store(ctx, qkv, self.n_heads, self.n_kv_heads, self.head_dim, cache, self.qk_norm_eps)
        attn_scale, floor_scale = self.position.query_temperature()
        out = torch.empty_like(q)
        self.attend(ctx, q, cache, out, attn_scale, floor_scale)
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
            if ctx.attn_tiles is not None:
                if ctx.n_attn_single_rows:
                    # the single decoded tokens of a mixed step go to the split-KV kernel, by their row list
                    self._split_kv(ctx, q, cache, out, attn_scale, floor_scale, ctx.attn_single_rows, ctx.n_attn_single_rows)
                tiles, n_tiles = ctx.attn_tiles, ctx.n_attn_tiles  # every request that brings more than one token
                if ctx.n_attn_tiles_big and self.head_dim in self.TC_HEAD_SIZES and K.attention_prefill_tc_supported(
                        q.dtype, self.n_heads, self.n_kv_heads, self.head_dim, cache.pages.shape[3]):
                    # long portions on the tcgen05 kernel (128-token tiles), the short ones below
                    K.attention_prefill_tc(q, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, out,
                                           ctx.attn_tiles_big, ctx.n_attn_tiles_big, self.scale, chunk, window,
                                           attn_scale, floor_scale, ctx.status)
                    tiles, n_tiles = ctx.attn_tiles_rest, ctx.n_attn_tiles_rest
                if n_tiles:
                    K.attention_prefill(q, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, out, tiles,
                                        n_tiles, self.scale, chunk, window, attn_scale, floor_scale, ctx.status)
                return
        K.attention_generic(q, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, out, self.scale,
                            self.chunk or 0, self.window or 0, attn_scale, floor_scale, ctx.status)


register_part("mixer", "paged_attention", PagedAttention)
