"""Norm parts."""

from __future__ import annotations

import torch

from ..kernels import api as K
from .base import Norm, StepContext, register_part


class RMSNorm(Norm):
    """out = weight * x / sqrt(mean(x^2) + eps), mean and division in float32
    (llama4/llama4_jax/model.py:885-888).  ``weight`` None = weightless."""

    kernel_libraries = ("elementwise",)

    def __init__(self, weight: torch.Tensor | None, eps: float):
        self.weight = None if weight is None else weight.to(torch.float32).contiguous()
        self.eps = float(eps)

    def forward(self, ctx: StepContext, x, delta, *, out_dtype, want_f32=False, row_index=None):
        n = x.shape[0] if row_index is None else row_index.numel()
        out = torch.empty((n, x.shape[1]), dtype=out_dtype, device=x.device)
        out32 = torch.empty((n, x.shape[1]), dtype=torch.float32, device=x.device) if want_f32 else None
        K.add_rmsnorm(x, delta, self.weight, self.eps, out, out32, row_index)
        return out, out32


register_part("norm", "rms", RMSNorm)
