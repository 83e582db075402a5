"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and has no model code of its own: it drives the same model, step function,
cache manager and kernels that generation uses.  Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step that wants logits, ``<out>/<step>.f32`` holds them as little-endian float32 [wanted, vocab]
in the order of the entries and of each ``want``.  After every step a line ``done <step>`` goes to
standard output.  The reference has nothing like it (its tests only check that prefill and two decode
steps run, llama4/tests/test_model.py:129-143).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each rounded up to whole pages)")
    ap.add_argument("--page-size", type=int, default=64, help="tokens per cache page")
    ap.add_argument("--max-requests", type=int, default=16, help="most requests live at a time")
    args = ap.parse_args(argv)

    print("[trace_run] loading torch and the model ...", file=sys.stderr, flush=True)
    import torch

    from ..loading import load_model
    from .engine import Engine, StepEntry

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 3
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    model = load_model(args.model, args.dtype, "cuda")
    # --max-tokens counts each live request rounded up to a multiple of 64 tokens.  Pages that are larger than
    # that round a request up further: by up to (page - 64) tokens for each live request.
    ps = args.page_size
    pool_tokens = -(-args.max_tokens // max(ps, 64)) * max(ps, 64) + args.max_requests * max(ps - 64, 0)
    engine = Engine(model, max_tokens=pool_tokens, page_size=args.page_size, max_slots=args.max_requests,
                    max_seq_len=pool_tokens)
    print("[trace_run] ready", file=sys.stderr, flush=True)
    slots: dict[str, int] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.new_request()
            if e.get("tokens"):  # an entry without tokens only makes the request known
                entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                arr = logits.to("cpu").numpy().astype("<f4", copy=False)
                tmp = out_dir / f"{step}.f32.tmp"
                arr.tofile(tmp)
                tmp.rename(out_dir / f"{step}.f32")
            engine.check_status()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                engine.finish(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
