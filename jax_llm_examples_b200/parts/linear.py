"""Matrix products y = a W^T for stored Linear weights W [out, in].

bfloat16 activations with bfloat16 weights go to the library GEMM (cuBLAS through torch), as the
reference leaves its dense products to its library (XLA dot_general, llama4/llama4_jax/model.py:
907-909, 952-954, 1146-1152, 1204).  Everything else runs on this package's own 32-bit FMA kernel:
the true 32-bit path (so that no reduced-precision matrix mode is possible), and weights that are
stored in 32-bit while activations are bfloat16.
"""

from __future__ import annotations

import torch

from ..kernels import api as K


def linear(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """a: [M, K]; w: [N, K]; returns [M, N] in out_dtype (float32 accumulation)."""
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if out_dtype == torch.bfloat16:
            return torch.mm(a, w.t())
        return torch.mm(a, w.t(), out_dtype=torch.float32)
    out = torch.empty((a.shape[0], w.shape[0]), dtype=out_dtype, device=a.device)
    K.gemm_simt(a, w, out)
    return out


def grouped_linear(a_sorted: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Rows [offsets[e], offsets[e+1]) of a_sorted times w[e]^T.  w: [E, N, K]."""
    out = torch.empty((a_sorted.shape[0], w.shape[1]), dtype=out_dtype, device=a_sorted.device)
    K.gemm_simt(a_sorted, w, out, offsets)
    return out
