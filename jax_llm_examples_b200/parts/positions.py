"""Position-encoding parts."""

from __future__ import annotations

import math

import torch

from ..kernels import api as K
from .base import LayerCache, PositionEncoding, Rows, StepContext, as_rows, register_part


def llama3_scaled_frequencies(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """Rotary frequencies f_j = theta^(-2j/dh) with the llama3 wavelength correction
    (llama4/llama4_jax/model.py:654-672, 706-709), evaluated in float32 like the reference.

    ``scaling``: factor, low_freq_factor, high_freq_factor, original_max_position_embeddings, or None
    for no correction.  With high == low there is no medium band, so the interpolation of
    model.py:668 (a division by zero there) is not evaluated."""
    fraction = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    freq = 1.0 / (torch.tensor(theta, dtype=torch.float32) ** fraction)
    if scaling is None:
        return freq
    factor, low, high = float(scaling["factor"]), float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    wavelen = 2 * math.pi / freq
    scaled = torch.where(wavelen > orig / low, freq / factor, freq)
    if high != low:
        smooth = (orig / wavelen - low) / (high - low)
        medium = ~(wavelen < orig / high) & ~(wavelen > orig / low)
        scaled = torch.where(medium, (1 - smooth) * scaled / factor + smooth * scaled, scaled)
    return scaled


class _FusedEncoding(PositionEncoding):
    kernel_libraries = ("rope_kv",)
    accepts_partials = True
    inv_freq: torch.Tensor | None = None

    def encode_and_store(self, ctx: StepContext, qkv, n_heads, n_kv_heads, head_dim, cache: LayerCache, qk_norm_eps):
        rows = as_rows(qkv)
        q = torch.empty((ctx.n_tokens, n_heads, head_dim), dtype=ctx.runtime.dtype, device=rows.data.device)
        l2 = qk_norm_eps is not None and self.norm_applies
        K.rope_kv_store(rows.data, q, cache.pages if cache.writes else None, cache.block_table if cache.writes else None,
                        ctx.req_of_token, ctx.positions, self.inv_freq, l2, qk_norm_eps if l2 else 1.0, n_heads,
                        n_kv_heads, head_dim, ctx.status, rows.splits)
        return q


class InterleavedRope(_FusedEncoding):
    """Rotation of adjacent pairs (2j, 2j+1) by position * f_j (model.py:722-728); the weightless
    q/k norm, where the mixer has one, follows the rotation (model.py:915-917)."""

    norm_applies = True

    def __init__(self, inv_freq: torch.Tensor, device):
        self.inv_freq = inv_freq.to(device=device, dtype=torch.float32).contiguous()


class NoPositionWithTemperature(_FusedEncoding):
    """No rotation and no q/k norm (model.py:913-917 skip both on these layers).  Queries are scaled by
    1 + attn_scale * ln(1 + floor((p + 1) / floor_scale)); attn_scale = 0 turns that off.  The scale is
    applied to the scores in float32 inside the attention kernel."""

    norm_applies = False

    def __init__(self, attn_scale: float = 0.0, floor_scale: float = 1.0):
        self.attn_scale, self.floor_scale = float(attn_scale), float(floor_scale)

    def query_temperature(self):
        return (self.attn_scale, self.floor_scale)


register_part("position", "interleaved_rope", InterleavedRope)
register_part("position", "none_with_temperature", NoPositionWithTemperature)


class UnfusedEncoding(PositionEncoding):
    """Base for an encoding that is written as a function of (q, k, positions): subclasses give
    ``transform``; the rows are then stored with the plain page-write kernel.  The q/k norm is the
    subclass's own business (``qk_norm_eps`` is handed to ``transform``)."""

    kernel_libraries = ("rope_kv",)

    def transform(self, ctx: StepContext, q: torch.Tensor, k: torch.Tensor, qk_norm_eps: float | None):
        raise NotImplementedError

    def encode_and_store(self, ctx: StepContext, qkv, n_heads, n_kv_heads, head_dim, cache: LayerCache, qk_norm_eps):
        n = qkv.shape[0]
        q = qkv[:, : n_heads * head_dim].reshape(n, n_heads, head_dim)
        k = qkv[:, n_heads * head_dim: (n_heads + n_kv_heads) * head_dim].reshape(n, n_kv_heads, head_dim)
        v = qkv[:, (n_heads + n_kv_heads) * head_dim:].reshape(n, n_kv_heads, head_dim)
        q, k = self.transform(ctx, q, k, qk_norm_eps)
        if cache.writes:
            K.kv_store(k.to(qkv.dtype).contiguous(), v.contiguous(), cache.pages, cache.block_table, ctx.req_of_token,
                       ctx.positions, ctx.status)
        return q.to(qkv.dtype).contiguous()
