"""Norm parts."""

from __future__ import annotations

import torch

from ..kernels import api as K
from .base import Norm, RowSum, StepContext, as_rows, register_part


class RMSNorm(Norm):
    """out = weight * x / sqrt(mean(x^2) + eps), mean and division in float32
    (llama4/llama4_jax/model.py:885-888).  ``weight`` None = weightless.  The residual sum x += delta
    runs in the same kernel, and so can the router of a following routed feed-forward."""

    kernel_libraries = ("elementwise",)
    fuses_router = True
    FUSED_ROUTER_MAX_ROWS = 64  # above this many rows (bfloat16) the router runs as its own many-rows kernel

    def __init__(self, weight: torch.Tensor | None, eps: float):
        self.weight = None if weight is None else weight.to(torch.float32).contiguous()
        self.eps = float(eps)

    def forward(self, ctx: StepContext, x, delta, *, out_dtype, want_f32=False, row_index=None, router=None):
        n = x.shape[0] if row_index is None else row_index.numel()
        dev = x.device
        out = torch.empty((n, x.shape[1]), dtype=out_dtype, device=dev)
        out32 = torch.empty((n, x.shape[1]), dtype=torch.float32, device=dev) if want_f32 else None
        # a sum of terms (an expert layer's rows still in expert order) is added term by term in the kernel
        # (the kernel takes so many terms, rows per token and partials; beyond that the sum is made by its producer)
        if isinstance(delta, RowSum) and len(delta.terms) <= K.DELTA_MAX_TERMS and all(t.k <= 16 for t in delta.terms) and \
                sum((t.k if t.index is not None else 1) * t.splits for t in delta.terms) <= K.DELTA_MAX_STREAMS:
            terms = [(t.data, t.splits, t.index, t.k, t.base) for t in delta.terms]
        else:
            d = as_rows(delta)
            terms = None if d is None else [(d.data, d.splits, None, 1, 0)]
        routing = None
        w_router = idx = wt = None
        unfused = False
        if router is not None and x.shape[1] <= 16384:
            w_router, k, *offer = router
            idx = torch.empty((n, k), dtype=torch.int32, device=dev)
            wt = torch.empty((n, k), dtype=torch.float32, device=dev)
            routing = (idx, wt)
            # Prompt portions in bfloat16: the router as a kernel of its own that shares each router row among
            # eight tokens (the fused kernel would fetch all router weights once per token).  The 32-bit path
            # keeps the fused kernel at every size: its sums must not depend on the batch.
            unfused = out_dtype == torch.bfloat16 and n > self.FUSED_ROUTER_MAX_ROWS and x.shape[1] % 4 == 0
            if unfused and out32 is None:
                out32 = torch.empty((n, x.shape[1]), dtype=torch.float32, device=dev)
        # a decode step's few rows: the kernel can also sort the choices and gather the rows for the experts
        dispatch = None
        if routing is not None and not unfused and offer and offer[0] is not None and row_index is None \
                and out_dtype == torch.bfloat16 and n <= K.DISPATCH_MAX_ROWS and n * k <= K.DISPATCH_MAX_PAIRS:
            dispatch = offer[0](ctx, n)
        did = K.add_rmsnorm(x, terms, self.weight, self.eps, out, out32, row_index, 1, None if unfused else w_router, idx, wt,
                            dispatch)
        if did:
            routing = (idx, wt, dispatch)
        if unfused:
            K.router(out32, w_router, idx, wt, many_rows=True)
        return out, out32, routing


register_part("norm", "rms", RMSNorm)
