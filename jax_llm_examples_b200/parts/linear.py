"""Matrix products y = a W^T for stored Linear weights W [out, in].

Which kernel runs:

* bfloat16 activations and weights, few rows (a decode step) or row groups (routed experts): this
  package's tcgen05 weight-streaming kernel (``csrc/gemm_stream.cu``), with K cut across blocks when
  the output is too narrow to fill the GPU.  The reference has its own kernel at exactly this place
  (llama4/llama4_jax/decode_ragged_dot.py).
* bfloat16, many rows, one group (prompt portions through the dense projections): the library GEMM
  (cuBLAS through torch), as the reference leaves its dense products to its library (XLA dot_general,
  llama4/llama4_jax/model.py:907-909, 952-954, 1146-1152, 1204).
* anything 32-bit (the true 32-bit path; weights stored in 32-bit under bfloat16 activations; K that
  is no multiple of 8): the 32-bit FMA kernel (``csrc/gemm_simt.cu``), so that no reduced-precision
  matrix mode is possible there.
"""

from __future__ import annotations

import torch

from ..kernels import api as K
from .base import StepContext

STREAM_MAX_ROWS = 256  # above this a dense product is compute-bound and goes to the library
_SM_COUNT = 148


def _splits_for(n_out: int, k: int) -> int:
    """K cuts so that about two blocks per SM stream weights; each cut keeps at least 512 of K."""
    tiles = -(-n_out // 128)
    want = -(-2 * _SM_COUNT // tiles)
    return max(1, min(want, k // 512, 8))


def linear(ctx: StepContext, a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """a: [M, K]; w: [N, K]; returns [M, N] in out_dtype (float32 accumulation)."""
    M, N = a.shape[0], w.shape[0]
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if M <= STREAM_MAX_ROWS and K.gemm_stream_supported(a, w):
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
            splits = _splits_for(N, a.shape[1])
            scratch = ctx.workspace.get("splitk", splits * M * N, torch.float32) if splits > 1 else None
            K.gemm_stream(a, w, out, ctx.status, splits=splits, scratch=scratch)
            return out
        if out_dtype == torch.bfloat16:
            return torch.mm(a, w.t())
        return torch.mm(a, w.t(), out_dtype=torch.float32)
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    K.gemm_simt(a, w, out)
    return out


def grouped_linear(ctx: StepContext, a_sorted: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor,
                   out_dtype: torch.dtype) -> torch.Tensor:
    """Rows [offsets[e], offsets[e+1]) of a_sorted times w[e]^T.  w: [E, N, K]."""
    rows, E = a_sorted.shape[0], w.shape[0]
    out = torch.empty((rows, w.shape[1]), dtype=out_dtype, device=a_sorted.device)
    if K.gemm_stream_supported(a_sorted, w):
        hint = min(rows, 2 * -(-rows // E))  # groups are uneven: tile for twice the mean
        K.gemm_stream(a_sorted, w, out, ctx.status, offsets=offsets, rows_hint=hint)
    else:
        K.gemm_simt(a_sorted, w, out, offsets)
    return out
