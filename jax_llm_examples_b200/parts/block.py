"""The arrangement of parts in a layer."""

from __future__ import annotations

import torch

from ..tracing import scope
from .base import Block, FeedForward, LayerCache, Mixer, Norm, StepContext, register_part


class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += feed_forward(norm2(x))  (llama4/llama4_jax/model.py:1156-1183).

    The residual sums are done in float32 inside the following norm's kernel: a block returns its
    last delta unadded, and the next block's first norm (or the model's final norm) adds it."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, feed_forward: FeedForward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def sub_parts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward)

    def forward(self, ctx: StepContext, x: torch.Tensor, delta, cache: LayerCache) -> torch.Tensor:
        dt = ctx.runtime.dtype
        with scope("attn_pre_norm"):  # the reference's names (model.py:1169-1180); each norm also adds the residual
            h = self.norm1.forward(ctx, x, delta, out_dtype=dt)[0]
        a = self.mixer.forward(ctx, h, cache)
        want32 = self.feed_forward.needs_f32_input
        router = self.feed_forward.router_request() if self.norm2.fuses_router else None
        with scope("attn_post_norm"):
            h, h32, routing = self.norm2.forward(ctx, x, a, out_dtype=dt, want_f32=want32, router=router)
        with scope("ffn"):
            return self.feed_forward.forward(ctx, h, h32, routing)


register_part("block", "pre_norm", PreNormBlock)
