"""Python face of the CUDA kernel libraries: loads them with ctypes and launches on torch's
current stream.  There is no fallback: a missing compiler, a failed build or a missing GPU
raises.  Every launch through this module is counted (``launch_count``)."""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from .. import tracing
from . import build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

STATUS_BITS = {
    1: "a block-table entry pointed outside the page pool",
    2: "a token id was outside the vocabulary",
    4: "a routed expert index was outside the expert count",
    8: "a bounded wait inside a kernel gave up",
}


class KernelError(RuntimeError):
    pass


_libs: dict[str, ctypes.CDLL] = {}
_launches = 0


def launch_count() -> int:
    return _launches


_sm_counts: dict[int, int] = {}


def sm_count() -> int:
    """Multiprocessors of the current device (asked once per device)."""
    dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return n


def library(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is None:
        path = build.ensure_built([name])[name]
        lib = ctypes.CDLL(str(path))
        lib.jlx_last_error.restype = ctypes.c_char_p
        _libs[name] = lib
    return lib


def preload(names) -> None:
    """Builds (in parallel) and loads the named libraries."""
    build.ensure_built(list(names))
    for n in names:
        library(n)


def loaded_libraries() -> list[str]:
    return sorted(_libs)


def code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"element type {dtype} is not supported by the kernels (float32, bfloat16)") from None


def _ptr(t: torch.Tensor | None):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a kernel was given a tensor that is not on the GPU; there is no CPU path")
    return c_void_p(t.data_ptr())


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _run(libname: str, fn: str, *args) -> None:
    global _launches
    lib = library(libname)
    timer = tracing.current_timer()
    if timer is None:
        rc = getattr(lib, fn)(*args)
    else:  # Generator(profile="kernels"): CUDA events around the launch
        rc_box = []
        timer.around(fn, lambda: rc_box.append(getattr(lib, fn)(*args)))
        rc = rc_box[0]
    if rc != 0:
        raise KernelError(f"{fn}: {lib.jlx_last_error().decode()}")
    _launches += 1


def _contig(*ts: torch.Tensor | None) -> None:
    for t in ts:
        if t is not None and not t.is_contiguous():
            raise KernelError("a kernel was given a tensor that is not contiguous")


# ------------------------------------------------------------------------------ elementwise
def embed(ids: torch.Tensor, table: torch.Tensor, x_out: torch.Tensor, status: torch.Tensor) -> None:
    _contig(ids, table, x_out)
    V, D = table.shape
    _run("elementwise", "jlx_embed", _ptr(ids), _ptr(table), c_int(code(table.dtype)), _ptr(x_out),
         c_int(ids.numel()), c_int(D), c_int(V), _ptr(status), _stream())


def _splits(t: torch.Tensor | None, splits: int) -> tuple[int, int]:
    """(split count, elements between partials) of a tensor that may hold split-K partials [splits, ...]."""
    if t is None or splits <= 1:
        return 1, 0
    return splits, t.numel() // splits


DELTA_MAX_TERMS = 3
DELTA_MAX_STREAMS = 64  # rows x split-K partials that one token may add (csrc/elementwise.cu)
DISPATCH_MAX_ROWS, DISPATCH_MAX_PAIRS = 16, 64  # csrc/elementwise.cu


class _DeltaTerm(ctypes.Structure):
    _fields_ = [("p", c_void_p), ("stride", c_longlong), ("index", c_void_p), ("splits", c_int), ("k", c_int), ("base", c_int)]


class _DeltaSpec(ctypes.Structure):
    _fields_ = [("n", c_int), ("t", _DeltaTerm * DELTA_MAX_TERMS)]


class _DispatchArgs(ctypes.Structure):  # DispatchArgs in csrc/elementwise.cu
    _fields_ = [("counter", c_void_p), ("offsets", c_void_p), ("sorted_pair", c_void_p), ("sorted_pos", c_void_p),
                ("tile_list", c_void_p), ("n_tiles", c_void_p), ("a_sorted", c_void_p), ("extra_rows", c_int),
                ("tile_rows", c_int), ("status", c_void_p)]


def add_rmsnorm(x: torch.Tensor, delta, gamma: torch.Tensor | None, eps: float,
                out: torch.Tensor | None, out32: torch.Tensor | None = None, row_index: torch.Tensor | None = None,
                delta_splits: int = 1, w_router: torch.Tensor | None = None, topk_idx: torch.Tensor | None = None,
                topk_w: torch.Tensor | None = None, dispatch=None) -> bool:
    """x (+= delta); out = gamma * x / sqrt(mean(x^2) + eps).  ``delta``: a float32 tensor that may hold
    ``delta_splits`` split-K partials [splits, N, D], added in order; or a list of up to DELTA_MAX_TERMS terms
    ``(data, splits, index, k, base)`` added in the order given: of the float32 partials ``data`` [splits, rows, D]
    token r takes row ``base + r`` or, with ``index`` (int32 [N * k]), the k rows ``index[r * k + j]``.
    With row_index, row n reads source row row_index[n] and x is not written back.  With w_router [E, D] the token
    is routed in the same kernel: topk_idx / topk_w [N, k].  ``dispatch`` (with w_router; an object with the tensors
    counter, offsets, sorted_pair, sorted_pos, a_sorted, status, the optional pair tiles = (tile_list, n_tiles) and
    the numbers extra_rows, tile_rows): what ``expert_sort`` and ``permute_scale`` would write next; the kernel does
    their work too when the step is small enough for that, and the call returns whether it did."""
    terms = [] if delta is None else (list(delta) if isinstance(delta, (list, tuple)) else [(delta, delta_splits, None, 1, 0)])
    _contig(x, gamma, out, out32, row_index, w_router, topk_idx, topk_w, *(t[0] for t in terms), *(t[2] for t in terms))
    D = x.shape[-1]
    n = row_index.numel() if row_index is not None else x.numel() // D
    if x.dtype != torch.float32 or any(t[0].dtype != torch.float32 for t in terms):
        raise KernelError("add_rmsnorm: the residual stream must be float32")
    if gamma is not None and gamma.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the norm weight must be float32")
    if len(terms) > DELTA_MAX_TERMS:
        raise KernelError(f"add_rmsnorm: {len(terms)} terms to add; up to {DELTA_MAX_TERMS} are supported")
    spec = _DeltaSpec()
    spec.n = len(terms)
    for q, (data, splits, index, k_rows, base) in enumerate(terms):
        sp, stride = _splits(data, splits)
        spec.t[q].p, spec.t[q].stride, spec.t[q].splits = data.data_ptr(), stride, sp
        spec.t[q].index, spec.t[q].k, spec.t[q].base = (index.data_ptr() if index is not None else None), k_rows, base
    E = k = 0
    if w_router is not None:
        if w_router.dtype != torch.float32 or topk_idx is None or topk_w is None:
            raise KernelError("router: float32 weight and outputs are needed")
        E, k = w_router.shape[0], topk_idx.shape[1]
    dp, did = None, c_int(0)
    if dispatch is not None and w_router is not None:
        tile_list, n_tiles = dispatch.tiles if dispatch.tiles is not None else (None, None)
        _contig(dispatch.offsets, dispatch.sorted_pair, dispatch.sorted_pos, dispatch.a_sorted, tile_list, n_tiles)
        if out is None or dispatch.a_sorted.dtype != out.dtype:
            raise KernelError("add_rmsnorm: the gathered rows must have the output's type")
        dp = _DispatchArgs(_ptr(dispatch.counter), _ptr(dispatch.offsets), _ptr(dispatch.sorted_pair), _ptr(dispatch.sorted_pos),
                           _ptr(tile_list), _ptr(n_tiles), _ptr(dispatch.a_sorted), dispatch.extra_rows,
                           dispatch.tile_rows if tile_list is not None else 0, _ptr(dispatch.status))
    _run("elementwise", "jlx_add_rmsnorm", _ptr(x), ctypes.byref(spec) if terms else None, _ptr(gamma), c_float(eps),
         _ptr(out), c_int(code(out.dtype) if out is not None else F32), _ptr(out32), _ptr(row_index), c_int(n), c_int(D),
         _ptr(w_router), c_int(E), c_int(k), _ptr(topk_idx), _ptr(topk_w), ctypes.byref(dp) if dp is not None else None,
         ctypes.byref(did), _stream())
    return bool(did.value)


def silu_mul(gu: torch.Tensor, out: torch.Tensor, splits: int = 1, interleaved: bool = False) -> None:
    """out = silu(gate) * up.  gu: [rows, 2F] (or ``splits`` float32 partials [splits, rows, 2F]), laid out
    [gate, up] or, interleaved, in blocks of [16 gate, 16 up]."""
    _contig(gu, out)
    rows, F = out.shape
    sp, stride = _splits(gu, splits)
    _run("elementwise", "jlx_silu_mul", _ptr(gu), c_int(code(gu.dtype)), c_int(sp), c_longlong(stride), _ptr(out),
         c_int(code(out.dtype)), c_int(rows), c_int(F), c_int(int(interleaved)), _stream())


# ------------------------------------------------------------------- position encoding + cache
def rope_kv_store(qkv: torch.Tensor, q_out: torch.Tensor, pages: torch.Tensor | None, block_table: torch.Tensor | None,
                  req_of_token: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor | None, l2norm: bool,
                  eps: float, Hq: int, Hkv: int, dh: int, status: torch.Tensor, splits: int = 1) -> None:
    """qkv: [N, (Hq + 2 Hkv) * dh] projected rows, or ``splits`` float32 partials of them.
    pages: [num_pages, 2, Hkv, page_size, dh] or None (a layer that writes no cache)."""
    _contig(qkv, q_out, pages, block_table, inv_freq)
    store = pages is not None
    N = q_out.shape[0]
    sp, stride = _splits(qkv, splits)
    _run("rope_kv", "jlx_rope_kv_store", _ptr(qkv), c_int(code(qkv.dtype)), c_int(sp), c_longlong(stride), _ptr(q_out),
         _ptr(pages), c_int(code(q_out.dtype)), _ptr(block_table), c_int(block_table.shape[1] if store else 0),
         _ptr(req_of_token), _ptr(positions), _ptr(inv_freq), c_int(int(l2norm)), c_float(eps), c_int(N), c_int(Hq),
         c_int(Hkv), c_int(dh), c_int(pages.shape[3] if store else 0), c_int(pages.shape[0] if store else 0),
         c_int(int(store)), _ptr(status), _stream())


def kv_store(k: torch.Tensor, v: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
             req_of_token: torch.Tensor, positions: torch.Tensor, status: torch.Tensor) -> None:
    _contig(k, v, pages, block_table)
    N, Hkv, dh = k.shape
    _run("rope_kv", "jlx_kv_store", _ptr(k), _ptr(v), _ptr(pages), c_int(code(k.dtype)), _ptr(block_table),
         c_int(block_table.shape[1]), _ptr(req_of_token), _ptr(positions), c_int(N), c_int(Hkv), c_int(dh),
         c_int(pages.shape[3]), c_int(pages.shape[0]), _ptr(status), _stream())


# ---------------------------------------------------------------------------------- attention
def attention_generic(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, req_of_token: torch.Tensor,
                      positions: torch.Tensor, out: torch.Tensor, scale: float, chunk: int, window: int,
                      attn_scale: float, floor_scale: float, status: torch.Tensor) -> None:
    """q: [N, Hq, dh]; pages: [P, 2, Hkv, page, dh]; out: [N, Hq, dh]."""
    _contig(q, pages, block_table, out)
    N, Hq, dh = q.shape
    P, _, Hkv, page_size, dh2 = pages.shape
    if dh2 != dh or pages.dtype != q.dtype:
        raise KernelError("attention: cache pages and queries disagree in head size or element type")
    _run("attention_generic", "jlx_attention_generic", _ptr(q), _ptr(pages), c_int(code(q.dtype)), _ptr(block_table),
         c_int(block_table.shape[1]), _ptr(req_of_token), _ptr(positions), _ptr(out), c_int(N), c_int(Hq), c_int(Hkv),
         c_int(dh), c_int(page_size), c_int(P), c_float(scale), c_int(chunk), c_int(window), c_float(attn_scale),
         c_float(floor_scale), _ptr(status), _stream())


def attention_mma_supported(q_dtype: torch.dtype, Hq: int, Hkv: int, dh: int, decode: bool) -> bool:
    if q_dtype != torch.bfloat16:
        return False
    return bool(library("attention_mma").jlx_attention_mma_supported(c_int(Hq), c_int(Hkv), c_int(dh), c_int(int(decode))))


def attention_decode_plan(max_kv_len: int, chunk: int, window: int, pairs: int) -> tuple[int, int]:
    """(keys per split, splits) for a decode launch over `pairs` (request, KV head) pairs."""
    lib = library("attention_mma")
    keys = int(lib.jlx_attention_decode_split_keys(c_int(max_kv_len), c_int(chunk), c_int(window), c_int(pairs)))
    return keys, int(lib.jlx_attention_decode_splits(c_int(max_kv_len), c_int(chunk), c_int(window), c_int(keys)))


def attention_decode(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, req_of_token: torch.Tensor,
                     positions: torch.Tensor, out: torch.Tensor, scale: float, chunk: int, window: int, attn_scale: float,
                     floor_scale: float, part_o: torch.Tensor, part_ml: torch.Tensor, max_splits: int, split_keys: int,
                     status: torch.Tensor, rows: torch.Tensor | None = None, n_rows: int = 0) -> None:
    """Split-KV attention for one query token per request (tensor cores, bfloat16).
    part_o: float32 [N * Hq * max_splits * dh]; part_ml: float32 [N * Hq * max_splits * 2].
    rows / n_rows: work on these token rows only (int32, the first n_rows entries): the single decoded tokens of
    a step that also holds prompt portions; N is then n_rows."""
    _contig(q, pages, block_table, out, part_o, part_ml, rows)
    N, Hq, dh = q.shape
    if rows is not None:
        N = n_rows
    P, _, Hkv, page_size, _ = pages.shape
    if part_o.numel() < N * Hq * max_splits * dh or part_ml.numel() < N * Hq * max_splits * 2:
        raise KernelError("attention_decode: scratch for the partial results is too small")
    _run("attention_mma", "jlx_attention_decode", _ptr(q), _ptr(pages), _ptr(block_table), c_int(block_table.shape[1]),
         _ptr(req_of_token), _ptr(positions), _ptr(out), c_int(N), c_int(Hq), c_int(Hkv), c_int(dh), c_int(page_size),
         c_int(P), c_float(scale), c_int(chunk), c_int(window), c_float(attn_scale), c_float(floor_scale), _ptr(part_o),
         _ptr(part_ml), c_int(max_splits), c_int(split_keys), _ptr(rows), _ptr(status), _stream())


def attention_prefill(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, req_of_token: torch.Tensor,
                      positions: torch.Tensor, out: torch.Tensor, tiles: torch.Tensor, n_tiles: int, scale: float,
                      chunk: int, window: int, attn_scale: float, floor_scale: float, status: torch.Tensor) -> None:
    """Flash attention over the paged cache for prompt portions (tensor cores, bfloat16).
    tiles: int32 [n_tiles, 2] = (first token row, count <= 16), each within one request."""
    _contig(q, pages, block_table, out, tiles)
    N, Hq, dh = q.shape
    P, _, Hkv, page_size, _ = pages.shape
    _run("attention_mma", "jlx_attention_prefill", _ptr(q), _ptr(pages), _ptr(block_table), c_int(block_table.shape[1]),
         _ptr(req_of_token), _ptr(positions), _ptr(out), _ptr(tiles), c_int(n_tiles), c_int(Hq), c_int(Hkv), c_int(dh),
         c_int(page_size), c_int(P), c_float(scale), c_int(chunk), c_int(window), c_float(attn_scale),
         c_float(floor_scale), _ptr(status), _stream())


def attention_prefill_tc_supported(q_dtype: torch.dtype, Hq: int, Hkv: int, dh: int, page_size: int) -> bool:
    if q_dtype != torch.bfloat16:
        return False
    return bool(library("attention_tc").jlx_attention_prefill_tc_supported(c_int(Hq), c_int(Hkv), c_int(dh), c_int(page_size)))


def attention_prefill_tc(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, req_of_token: torch.Tensor,
                         positions: torch.Tensor, out: torch.Tensor, tiles: torch.Tensor, n_tiles: int, scale: float,
                         chunk: int, window: int, attn_scale: float, floor_scale: float, status: torch.Tensor) -> None:
    """Flash attention for prompt portions on tcgen05 (bfloat16, head size 128, pages of a multiple of 64).
    tiles: int32 [n_tiles, 2] = (first token row, count <= 128), each within one request; only the rows
    of these tiles are written."""
    _contig(q, pages, block_table, out, tiles)
    N, Hq, dh = q.shape
    P, _, Hkv, page_size, _ = pages.shape
    _run("attention_tc", "jlx_attention_prefill_tc", _ptr(q), _ptr(pages), _ptr(block_table), c_int(block_table.shape[1]),
         _ptr(req_of_token), _ptr(positions), _ptr(out), _ptr(tiles), c_int(n_tiles), c_int(N), c_int(Hq), c_int(Hkv),
         c_int(dh), c_int(page_size), c_int(P), c_float(scale), c_int(chunk), c_int(window), c_float(attn_scale),
         c_float(floor_scale), _ptr(status), _stream())


# ------------------------------------------------------------------------------------- GEMMs
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor | None = None) -> None:
    """out = a @ w^T.  a: [M, K]; w: [N, K], or [E, N, K] with row-group offsets [E + 1] on the device."""
    _contig(a, w, out, offsets)
    M, K = a.shape
    if offsets is None:
        N, E, stride = w.shape[0], 0, 0
    else:
        E, N = w.shape[0], w.shape[1]
        stride = N * K
    if w.shape[-1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm: shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _run("gemm_simt", "jlx_gemm_simt", _ptr(a), c_int(code(a.dtype)), _ptr(w), c_int(code(w.dtype)), _ptr(out),
         c_int(code(out.dtype)), c_int(M), c_int(N), c_int(K), c_longlong(K), c_longlong(K), c_longlong(N),
         _ptr(offsets), c_int(E), c_longlong(stride), _stream())


def gemm_stream_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[-1] % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


GEMM_PLAIN, GEMM_PARTIALS, GEMM_SWIGLU = 0, 1, 2


def gemm_stream_token_tile(rows_hint: int) -> int:
    """The token-tile width gemm_stream uses for this rows_hint."""
    return int(library("gemm_stream").jlx_gemm_stream_token_tile(c_int(rows_hint)))


def gemm_stream(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
                offsets: torch.Tensor | None = None, rows_hint: int = 0, splits: int = 1,
                scratch: torch.Tensor | None = None, mode: int = GEMM_PLAIN,
                tiles: tuple[torch.Tensor, torch.Tensor] | None = None, offsets_settled: bool = False) -> int:
    """a @ w^T on the tcgen05 tensor cores (bfloat16 in, float32 accumulate).  a: [M, K]; w: [N, K] or,
    with row-group offsets [E + 1], [E, N, K].
    GEMM_PLAIN: out [M, N] bfloat16 or float32; splits > 1 cuts K across blocks (scratch: float32
    [splits * M * N]) and adds the partials.  GEMM_PARTIALS: out is float32 [splits, M, N], left for the
    consumer to add.  GEMM_SWIGLU: w's rows are interleaved [16 gate, 16 up]; out [M, N / 2] =
    silu(gate) * up.  ``tiles`` = (tile_list, n_tiles) from expert_sort for the same rows_hint.
    ``offsets_settled``: the kernel launched just before this call on the stream was a grouped gemm_stream over the
    same offsets and tiles (this one then finds its tile and asks for its weights without waiting for that one).
    Returns the split count used."""
    _contig(a, w, out, offsets, scratch)
    M, K = a.shape
    E = w.shape[0] if offsets is not None else 0
    N = w.shape[-2]
    if w.shape[-1] != K or (offsets is None) != (w.dim() == 2):
        raise KernelError(f"gemm_stream: shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}")
    want = {GEMM_PLAIN: M * N, GEMM_PARTIALS: splits * M * N, GEMM_SWIGLU: M * (N // 2)}[mode]
    if out.numel() < want:
        raise KernelError(f"gemm_stream: out has {out.numel()} elements, {want} are needed")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_stream: bfloat16 operands and a bfloat16 or float32 result are supported")
    if mode == GEMM_PLAIN and splits > 1 and (scratch is None or scratch.numel() < splits * M * N or scratch.dtype != torch.float32):
        raise KernelError("gemm_stream: split-K needs float32 scratch of splits * M * N elements")
    used = c_int(1)
    _run("gemm_stream", "jlx_gemm_stream", _ptr(a), _ptr(w), _ptr(out), c_int(int(out.dtype == torch.float32)), c_int(M),
         c_int(N), c_int(K), _ptr(offsets), c_int(E), c_int(rows_hint), c_int(splits), _ptr(scratch), c_int(mode),
         _ptr(tiles[0]) if tiles else None, _ptr(tiles[1]) if tiles else None, c_int(int(offsets_settled and offsets is not None)),
         ctypes.byref(used), _ptr(status), _stream())
    return used.value


# --------------------------------------------------------------------------------------- MoE
def router(h32: torch.Tensor, w_router: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor,
           scores_out: torch.Tensor | None = None, many_rows: bool = False) -> None:
    """Scores h32 @ w_router^T in 32-bit, top-k of the raw scores (lower index wins ties), weight = sigmoid.
    ``many_rows``: the kernel that shares each router row among eight tokens (for prompt portions; its sums
    run in another order than the one-token kernel's)."""
    _contig(h32, w_router, topk_idx, topk_w, scores_out)
    N, D = h32.shape
    E, k = w_router.shape[0], topk_idx.shape[1]
    if h32.dtype != torch.float32 or w_router.dtype != torch.float32:
        raise KernelError("router: scores are computed from float32 input and weight")
    _run("moe", "jlx_router", _ptr(h32), _ptr(w_router), _ptr(topk_idx), _ptr(topk_w), _ptr(scores_out), c_int(N),
         c_int(D), c_int(E), c_int(k), c_int(int(many_rows)), _stream())


def expert_sort(topk_idx: torch.Tensor, offsets: torch.Tensor, sorted_pair: torch.Tensor, sorted_pos: torch.Tensor,
                E: int, status: torch.Tensor, extra_rows: int = 0, tile_rows: int = 0,
                tile_list: torch.Tensor | None = None, n_tiles: torch.Tensor | None = None) -> None:
    """Counting sort of the (token, choice) pairs by expert.  offsets: [E + 1], or [E + 2] with extra_rows > 0:
    one more group of that many rows appended after the experts.  With tile_rows > 0 also the list of row
    tiles of that height that hold rows: tile_list int32 [(ceil(rows / tile_rows) + groups) * 2], n_tiles [1]."""
    _contig(topk_idx, offsets, sorted_pair, sorted_pos, tile_list, n_tiles)
    if offsets.numel() < E + 1 + (extra_rows > 0):
        raise KernelError("expert_sort: offsets too short")
    if tile_rows > 0:
        rows, groups = topk_idx.numel() + extra_rows, E + (extra_rows > 0)
        if tile_list is None or n_tiles is None or tile_list.numel() < 2 * (-(-rows // tile_rows) + groups):
            raise KernelError("expert_sort: tile list too short")
    _run("moe", "jlx_expert_sort", _ptr(topk_idx), _ptr(offsets), _ptr(sorted_pair), _ptr(sorted_pos),
         c_int(topk_idx.numel()), c_int(E), c_int(extra_rows), c_int(tile_rows), _ptr(tile_list), _ptr(n_tiles),
         _ptr(status), _stream())


def permute_scale(h32: torch.Tensor, sorted_pair: torch.Tensor, topk_w: torch.Tensor, a_sorted: torch.Tensor, k: int,
                  extra_rows: int = 0) -> None:
    """a_sorted[i] = weight * h32[token] in expert order; then extra_rows unscaled copies of h32's rows."""
    _contig(h32, sorted_pair, topk_w, a_sorted)
    P = a_sorted.shape[0] - extra_rows
    _run("moe", "jlx_permute_scale", _ptr(h32), _ptr(sorted_pair), _ptr(topk_w), _ptr(a_sorted),
         c_int(code(a_sorted.dtype)), c_int(P), c_int(extra_rows), c_int(h32.shape[1]), c_int(k), _stream())


def moe_combine(y_sorted: torch.Tensor, shared: torch.Tensor | None, sorted_pos: torch.Tensor, delta: torch.Tensor, k: int,
                shared_splits: int = 1, y_splits: int = 1, extra_base: int = -1) -> None:
    """delta = the sum of each token's expert rows (+ row extra_base + n of y: an appended shared group)
    (+ shared); y_sorted and shared may be split-K partials."""
    _contig(y_sorted, shared, sorted_pos, delta)
    N, D = delta.shape
    sp, stride = _splits(shared, shared_splits)
    ysp, ystride = _splits(y_sorted, y_splits)
    _run("moe", "jlx_moe_combine", _ptr(y_sorted), c_int(ysp), c_longlong(ystride), c_int(extra_base), _ptr(shared),
         c_int(sp), c_longlong(stride), _ptr(sorted_pos), _ptr(delta), c_int(N), c_int(D), c_int(k), _stream())


# ---------------------------------------------------------------------------------- sampling
def sample_max_top_k() -> int:
    return int(library("sampling").jlx_sample_max_top_k())


def argmax(logits: torch.Tensor, out: torch.Tensor, part_v: torch.Tensor, part_i: torch.Tensor) -> None:
    """out[m] = index of the largest logit (lowest index on ties).  part_v (float32), part_i (int32): [M * 32] scratch."""
    _contig(logits, out, part_v, part_i)
    if logits.dtype != torch.float32:
        raise KernelError("argmax: logits must be float32")
    M, V = logits.shape
    if part_v.numel() < 32 * M or part_i.numel() < 32 * M:
        raise KernelError("argmax: scratch too small")
    _run("sampling", "jlx_argmax", _ptr(logits), c_int(M), c_int(V), c_longlong(V), _ptr(part_v), _ptr(part_i), _ptr(out),
         _stream())


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor | None = None,
           top_k: torch.Tensor | None = None, streams: torch.Tensor | None = None,
           counters: torch.Tensor | None = None, seed: int = 0) -> None:
    """out[m] = argmax (temperature None or <= 1e-3) or a draw from softmax(logits / temperature)."""
    _contig(logits, out, temperature, top_k, streams, counters)
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    M, V = logits.shape
    _run("sampling", "jlx_sample", _ptr(logits), c_int(M), c_int(V), c_longlong(V), _ptr(temperature), _ptr(top_k),
         _ptr(streams), _ptr(counters), c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _ptr(out), _stream())
