"""Microbenchmarks of single kernels at model sizes, with the bytes and FLOPs they must move.

    python -m jax_llm_examples_b200.kernels.microbench attention_decode --batch 8 --context 8192
    python -m jax_llm_examples_b200.kernels.microbench attention_prefill --tokens 2048
    python -m jax_llm_examples_b200.kernels.microbench gemm --rows 8 --n 16384 --k 5120 [--experts 16] [--swiglu]

The reference benchmarks its kernels the same way, from ``__main__`` blocks in the kernel files
(llama4/llama4_jax/ragged_attention.py:299-418, llama4/llama4_jax/decode_ragged_dot.py:239-291).
Timing: CUDA events around one launch, after warm-up, with a write larger than L2 between launches;
the median of the repetitions is reported.  Sizes default to the Scout layer sizes.
"""

from __future__ import annotations

import argparse
import json
import random

import torch

from . import api as K


def _time(fn, reps: int, flush: torch.Tensor | None) -> float:
    for _ in range(3):
        fn()
    times = []
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return sorted(times)[len(times) // 2] * 1e-3


def _paged(batch: int, context: int, hkv: int, dh: int, page: int, dev: str):
    pages_per = -(-context // page)
    n_pages = batch * pages_per
    pages = (torch.randn(n_pages, 2, hkv, page, dh, device=dev) * 0.5).bfloat16()
    table = torch.arange(n_pages, device=dev, dtype=torch.int32).view(batch, pages_per).contiguous()
    return pages, table


def attention_decode(a) -> dict:
    dev = "cuda"
    pages, table = _paged(a.batch, a.context, a.kv_heads, a.head_dim, a.page_size, dev)
    q = torch.randn(a.batch, a.heads, a.head_dim, device=dev).bfloat16()
    out = torch.empty_like(q)
    pos = torch.full((a.batch,), a.context - 1, device=dev, dtype=torch.int32)
    req = torch.arange(a.batch, device=dev, dtype=torch.int32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    keys, splits = K.attention_decode_plan(a.context, a.chunk, 0, a.batch * a.kv_heads)
    if a.split_keys:
        keys, splits = a.split_keys, -(-a.context // a.split_keys) + 1
    part_o = torch.empty(a.batch * a.heads * splits * a.head_dim, device=dev)
    part_ml = torch.empty(a.batch * a.heads * splits * 2, device=dev)

    def run():
        K.attention_decode(q, pages, table, req, pos, out, a.head_dim ** -0.5, a.chunk, 0, 0.0, 1.0, part_o, part_ml, splits,
                           keys, status)

    t = _time(run, a.reps, _flush(a))
    nbytes = a.batch * a.context * 2 * a.kv_heads * a.head_dim * 2
    assert int(status) == 0
    return {"kernel": "attention_decode", "batch": a.batch, "context": a.context, "split_keys": keys, "splits": splits,
            "us": round(t * 1e6, 1), "GB": round(nbytes / 1e9, 3), "GB/s": round(nbytes / t / 1e9, 1)}


def attention_prefill(a) -> dict:
    dev = "cuda"
    T = a.tokens
    pages, table = _paged(1, T, a.kv_heads, a.head_dim, a.page_size, dev)
    q = torch.randn(T, a.heads, a.head_dim, device=dev).bfloat16()
    out = torch.empty_like(q)
    pos = torch.arange(T, device=dev, dtype=torch.int32)
    req = torch.zeros(T, device=dev, dtype=torch.int32)
    rows = 128 if a.tc else 16
    tiles = torch.tensor([(t, min(rows, T - t)) for t in range(0, T, rows)][::-1], device=dev, dtype=torch.int32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    fn = K.attention_prefill_tc if a.tc else K.attention_prefill

    def run():
        fn(q, pages, table, req, pos, out, tiles, tiles.shape[0], a.head_dim ** -0.5, a.chunk, 0, 0.0, 1.0, status)

    t = _time(run, a.reps, _flush(a))
    flops = 4 * a.heads * a.head_dim * T * (T + 1) / 2
    assert int(status) == 0
    return {"kernel": "attention_prefill_tc" if a.tc else "attention_prefill", "tokens": T, "us": round(t * 1e6, 1), "TFLOP": round(flops / 1e12, 4),
            "TFLOP/s": round(flops / t / 1e12, 1)}


def gemm(a) -> dict:
    dev = "cuda"
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    x = torch.randn(a.rows, a.k, device=dev).bfloat16()
    E = a.experts
    w = (torch.randn(max(E, 1), a.n, a.k, device=dev) * 0.05).bfloat16()
    offsets, used, tiles = None, 1, None
    hint = a.hint or (min(a.rows, 2 * -(-a.rows // E)) if E else 0)
    if E:
        # rows spread over the groups at random; the sort kernel gives the offsets and, as in the engine, the
        # list of row tiles that hold rows
        rng = random.Random(0)
        choice = torch.tensor([rng.randrange(E) for _ in range(a.rows)], device=dev, dtype=torch.int32).view(-1, 1)
        offsets = torch.empty(E + 1, device=dev, dtype=torch.int32)
        pair, pos = torch.empty(a.rows, device=dev, dtype=torch.int32), torch.empty(a.rows, device=dev, dtype=torch.int32)
        tile_rows = K.gemm_stream_token_tile(hint)
        tiles = (torch.empty(2 * (-(-a.rows // tile_rows) + E), device=dev, dtype=torch.int32), torch.empty(1, device=dev, dtype=torch.int32))
        K.expert_sort(choice, offsets, pair, pos, E, status, 0, tile_rows, *tiles)
        used = int((offsets[1:] > offsets[:-1]).sum())
    else:
        w = w[0]
    mode = K.GEMM_SWIGLU if a.swiglu else K.GEMM_PLAIN
    out = torch.empty(a.rows, a.n // 2 if a.swiglu else a.n, device=dev, dtype=torch.bfloat16 if a.swiglu else torch.float32)
    scratch = torch.empty(a.splits * a.rows * a.n, device=dev) if a.splits > 1 else None

    def run():
        K.gemm_stream(x, w, out, status, offsets=offsets, rows_hint=hint, splits=a.splits, scratch=scratch, mode=mode, tiles=tiles)

    t = _time(run, a.reps, _flush(a))
    nbytes = used * a.n * a.k * 2 + a.rows * a.k * 2 + out.numel() * out.element_size()
    flops = 2 * a.rows * a.n * a.k
    assert int(status) == 0
    return {"kernel": "gemm_stream", "rows": a.rows, "n": a.n, "k": a.k, "experts": E, "experts_used": used if E else None,
            "splits": a.splits, "swiglu": a.swiglu, "us": round(t * 1e6, 1), "GB/s": round(nbytes / t / 1e9, 1),
            "TFLOP/s": round(flops / t / 1e12, 1)}


def _flush(a):
    return None if a.no_flush else torch.empty(256 * 1024 * 1024 // 4, device="cuda")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="what", required=True)
    for name in ("attention_decode", "attention_prefill", "gemm"):
        p = sub.add_parser(name)
        p.add_argument("--reps", type=int, default=10)
        p.add_argument("--no-flush", action="store_true", help="do not flush L2 between launches")
        if name.startswith("attention"):
            p.add_argument("--heads", type=int, default=40)
            p.add_argument("--kv-heads", type=int, default=8)
            p.add_argument("--head-dim", type=int, default=128)
            p.add_argument("--page-size", type=int, default=64)
            p.add_argument("--chunk", type=int, default=0)
        if name == "attention_decode":
            p.add_argument("--batch", type=int, default=8)
            p.add_argument("--context", type=int, default=8192)
            p.add_argument("--split-keys", type=int, default=0, help="keys per split (a multiple of 64) instead of the planned size")
        if name == "attention_prefill":
            p.add_argument("--tokens", type=int, default=2048)
            p.add_argument("--tc", action="store_true", help="the tcgen05 kernel (128-token tiles) instead of the mma.sync one")
        if name == "gemm":
            p.add_argument("--rows", type=int, default=8)
            p.add_argument("--n", type=int, default=16384)
            p.add_argument("--k", type=int, default=5120)
            p.add_argument("--experts", type=int, default=0, help="0: one dense weight; else rows are spread over this many groups")
            p.add_argument("--splits", type=int, default=1)
            p.add_argument("--hint", type=int, default=0, help="rows per group that the token tile is sized for (0: twice the mean)")
            p.add_argument("--swiglu", action="store_true", help="fused SiLU(gate) * up epilogue")
    a = ap.parse_args(argv)
    print(json.dumps({"attention_decode": attention_decode, "attention_prefill": attention_prefill, "gemm": gemm}[a.what](a)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
