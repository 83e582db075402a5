"""Choosing the next token from float32 logits.

The reference's Llama 4 decodes by argmax (llama4/llama4_jax/model.py:1266, 1275); the repository's
sampler is ``sample_top`` (gpt_oss/gpt_oss_jax/model.py:1125-1147): softmax(logits / temp), the k
most likely tokens, a draw by inverse CDF, and argmax when temp <= 1e-3.  Both are here, on the GPU.
The random number of a draw is a function of (seed, the request's stream, the request's step), so a
request's tokens do not depend on what else is in the batch or on when it was scheduled.
"""

from __future__ import annotations

import dataclasses

import torch

from ..kernels import api as K


@dataclasses.dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0  # <= 1e-3: greedy
    top_k: int = 0  # 0: the whole vocabulary
    seed: int = 0  # varies this request's random stream (see stream_of); the run's own seed is the Sampler's
    max_new_tokens: int = 32
    eos_token_ids: tuple[int, ...] = ()

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")


def stream_of(request_id: int, params: SamplingParams) -> int:
    """The random stream of a request: its id, moved by the seed of its sampling parameters (seed 0: the id)."""
    return (request_id ^ (params.seed * 0x9E3779B97F4A7C15)) & 0x7FFFFFFFFFFFFFFF


class Sampler:
    """Samples one token per row of logits; one seed for the whole run."""

    def __init__(self, seed: int = 0):
        self.seed = int(seed)
        self._max_k: int | None = None
        self._part: tuple[torch.Tensor, torch.Tensor] | None = None

    def sample(self, logits: torch.Tensor, temperatures: list[float], top_ks: list[int], streams: list[int],
               counters: list[int]) -> torch.Tensor:
        """logits: [M, V] float32 on the GPU.  Returns int32 [M] on the GPU."""
        M = logits.shape[0]
        out = torch.empty(M, dtype=torch.int32, device=logits.device)
        if all(t <= 1e-3 for t in temperatures):
            if self._part is None or self._part[0].numel() < 32 * M or self._part[0].device != logits.device:
                self._part = (torch.empty(32 * max(M, 64), dtype=torch.float32, device=logits.device),
                              torch.empty(32 * max(M, 64), dtype=torch.int32, device=logits.device))
            K.argmax(logits, out, *self._part)
            return out
        if self._max_k is None:
            self._max_k = K.sample_max_top_k()
        if max(top_ks) > self._max_k:
            raise ValueError(f"top_k {max(top_ks)} is above the sampler's maximum {self._max_k}")
        dev = logits.device
        # one host->device copy: temperatures (as int bits), top_k, then streams and counters (uint64 as 2 x int32)
        t = torch.tensor(temperatures, dtype=torch.float32).to(dev, non_blocking=True)
        k = torch.tensor(top_ks, dtype=torch.int32).to(dev, non_blocking=True)
        s = torch.tensor([x & 0x7FFFFFFFFFFFFFFF for x in streams], dtype=torch.int64).to(dev, non_blocking=True)
        c = torch.tensor(counters, dtype=torch.int64).to(dev, non_blocking=True)
        K.sample(logits, out, t, k, s, c, self.seed)
        return out
