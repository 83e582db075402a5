"""Matrix products y = a W^T for stored Linear weights W [out, in].

Which kernel runs:

* bfloat16 activations and weights, few rows (a decode step) or row groups (routed experts): this
  package's tcgen05 weight-streaming kernel (``csrc/gemm_stream.cu``), with K cut across blocks when
  the output is too narrow to fill the GPU.  The reference has its own kernel at exactly this place
  (llama4/llama4_jax/decode_ragged_dot.py).  Its consumers can take the split-K partials as they are
  (:class:`Rows`) and it can apply SiLU(gate) * up in its epilogue.
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
from .base import Rows, StepContext

# Every product of this package accumulates in float32.  The library's bfloat16 GEMM may otherwise add its
# split-K partial sums in bfloat16 (torch's default lets it): switched off for the process when this package loads.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

STREAM_MAX_ROWS = 256  # above this a dense product is compute-bound and goes to the library


def _resident_blocks() -> int:
    """Blocks of the streaming kernel that the GPU holds at once (two per multiprocessor)."""
    return 2 * K.sm_count()


def _splits_for(n_out: int, k: int, groups: int = 1, partials: bool = True) -> int:
    """K cuts for a product that streams `groups` weight matrices of n_out rows.  Fewer blocks than the GPU
    holds at once: cut K so that one round of blocks fills it, and no more (a second, nearly empty round
    costs as much as the first).  More blocks than that: rounds cannot be avoided, so cut K to about 2048
    per block (half a megabyte of weights), which keeps the last, partly filled round short; but only where
    the consumer adds the partials itself (`partials`): a separate pass over them costs more than the tail.
    Each cut keeps at least 512 of K."""
    busy = -(-n_out // 128) * max(groups, 1)
    resident = _resident_blocks()
    want = resident // busy if busy <= resident else (k // 2048 if partials else 1)
    return max(1, min(want, k // 512, 8))


def _group_rows_hint(rows: int, groups: int, largest_group: int = 0) -> int:
    """Rows that a token tile should hold so that almost every group fits one tile: rows spread over the
    groups like a binomial, so mean + 2.5 sigma (the rare larger group takes a second tile); at least the
    size of a group known to be large."""
    mean = rows / max(groups, 1)
    return max(min(rows, int(mean + 2.5 * mean ** 0.5 + 1)), largest_group, 1)


def _streams(a: torch.Tensor, w: torch.Tensor, rows_limit: bool) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K.gemm_stream_supported(a, w)
            and (not rows_limit or a.shape[0] <= STREAM_MAX_ROWS))


def interleave_gate_up(w_gate_up: torch.Tensor) -> torch.Tensor:
    """[..., 2F, D] with gate rows then up rows -> the same rows in blocks of [16 gate, 16 up], the layout
    whose product the SwiGLU epilogue can finish inside one warp.  F must be a multiple of 16."""
    F = w_gate_up.shape[-2] // 2
    g = w_gate_up[..., :F, :].unflatten(-2, (F // 16, 16))
    u = w_gate_up[..., F:, :].unflatten(-2, (F // 16, 16))
    return torch.stack([g, u], dim=-3).flatten(-4, -2).contiguous()


def linear(ctx: StepContext, a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, partials: bool = False):
    """a: [M, K]; w: [N, K]; returns [M, N] in out_dtype (float32 accumulation).  With ``partials`` the
    result is :class:`Rows`: float32 split-K slices that the consumer adds when the streaming kernel ran,
    else one slice in out_dtype."""
    M, N = a.shape[0], w.shape[0]
    if _streams(a, w, True):
        splits = _splits_for(N, a.shape[1], partials=partials)
        if partials:
            out = torch.empty((splits, M, N), dtype=torch.float32, device=a.device)
            used = K.gemm_stream(a, w, out, ctx.status, splits=splits, mode=K.GEMM_PARTIALS)
            return Rows(out[:used], used)
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        scratch = ctx.workspace.get("splitk", splits * M * N, torch.float32) if splits > 1 else None
        K.gemm_stream(a, w, out, ctx.status, splits=splits, scratch=scratch)
        return out
    # not the streaming kernel: one complete result in the type asked for (a consumer of Rows takes any type)
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        out = torch.mm(a, w.t()) if out_dtype == torch.bfloat16 else torch.mm(a, w.t(), out_dtype=torch.float32)
    else:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        K.gemm_simt(a, w, out)
    return Rows(out, 1) if partials else out


def swiglu_linear(ctx: StepContext, a: torch.Tensor, w_gate_up: torch.Tensor, interleaved: bool,
                  out_dtype: torch.dtype) -> torch.Tensor:
    """silu(a Wg^T) * (a Wu^T) for stacked [2F, K] weights: in the product's epilogue where the streaming
    kernel runs and the rows are interleaved, else a product followed by the activation kernel."""
    M, F = a.shape[0], w_gate_up.shape[0] // 2
    act = torch.empty((M, F), dtype=out_dtype, device=a.device)
    if interleaved and _streams(a, w_gate_up, True):
        K.gemm_stream(a, w_gate_up, act, ctx.status, mode=K.GEMM_SWIGLU)
        return act
    gu = linear(ctx, a, w_gate_up, out_dtype)
    K.silu_mul(gu, act, interleaved=interleaved)
    return act


def group_rows_hint(rows: int, groups: int, largest_group: int = 0) -> int:
    return _group_rows_hint(rows, groups, largest_group)


def grouped_linear(ctx: StepContext, a_sorted: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor,
                   out_dtype: torch.dtype, partials: bool = False, largest_group: int = 0, tiles=None, after_grouped: bool = False):
    """Rows [offsets[e], offsets[e+1]) of a_sorted times w[e]^T.  w: [E, N, K].  With ``partials`` the result
    is float32 :class:`Rows`; few rows (few groups in use) then get K cut across blocks to fill the GPU.
    ``after_grouped``: a_sorted was made by the call just before this one, ``grouped_swiglu_linear`` over the same
    offsets and tiles, which ran as one streaming product (``grouped_swiglu_streams``; see ``K.gemm_stream``)."""
    rows, E, N = a_sorted.shape[0], w.shape[0], w.shape[1]
    if _streams(a_sorted, w, False):
        hint = _group_rows_hint(rows, E, largest_group)
        if partials:
            # at most min(E, rows) groups have rows, and so many weight matrices are streamed
            splits = _splits_for(N, a_sorted.shape[1], min(E, rows)) if rows <= STREAM_MAX_ROWS else 1
            out = torch.empty((splits, rows, N), dtype=torch.float32, device=a_sorted.device)
            used = K.gemm_stream(a_sorted, w, out, ctx.status, offsets=offsets, rows_hint=hint, splits=splits, mode=K.GEMM_PARTIALS,
                                 tiles=tiles, offsets_settled=after_grouped)
            return Rows(out[:used], used)
        out = torch.empty((rows, N), dtype=out_dtype, device=a_sorted.device)
        K.gemm_stream(a_sorted, w, out, ctx.status, offsets=offsets, rows_hint=hint, tiles=tiles, offsets_settled=after_grouped)
        return out
    out = torch.empty((rows, N), dtype=torch.float32 if partials else out_dtype, device=a_sorted.device)
    K.gemm_simt(a_sorted, w, out, offsets)
    return Rows(out, 1) if partials else out


def grouped_swiglu_streams(a_sorted: torch.Tensor, w_gate_up: torch.Tensor, interleaved: bool) -> bool:
    """Whether ``grouped_swiglu_linear`` runs as ONE streaming product (activation in its epilogue), nothing after it."""
    return interleaved and _streams(a_sorted, w_gate_up, False)


def grouped_swiglu_linear(ctx: StepContext, a_sorted: torch.Tensor, w_gate_up: torch.Tensor, offsets: torch.Tensor,
                          interleaved: bool, out_dtype: torch.dtype, largest_group: int = 0, tiles=None) -> torch.Tensor:
    """``largest_group``: rows of a group known to be large (a shared expert's), so that one tile holds it."""
    rows, E, F = a_sorted.shape[0], w_gate_up.shape[0], w_gate_up.shape[1] // 2
    act = torch.empty((rows, F), dtype=out_dtype, device=a_sorted.device)
    if grouped_swiglu_streams(a_sorted, w_gate_up, interleaved):
        hint = _group_rows_hint(rows, E, largest_group)
        K.gemm_stream(a_sorted, w_gate_up, act, ctx.status, offsets=offsets, rows_hint=hint, mode=K.GEMM_SWIGLU, tiles=tiles)
        return act
    gu = grouped_linear(ctx, a_sorted, w_gate_up, offsets, out_dtype)
    K.silu_mul(gu, act, interleaved=interleaved)
    return act
