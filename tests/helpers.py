"""Shared by the tests: tiny model folders, the plain implementation's logits, trace families."""

from __future__ import annotations

import functools
import json
import os
import random
from pathlib import Path

import numpy as np
import torch

from tests.plain import llama4_plain as plain

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# A third tiny configuration, for the tensor-core kernels (head size 64, 3 query heads per KV head): the chunk
# (80) is no multiple of the key tile (64) or of the test page size (16); MoE layers are given as a list;
# llama3 scaling has equal low and high factors (no medium band).
TINY_C = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "num_hidden_layers": 5, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64,
    "moe_layers": [0, 2, 3], "num_local_experts": 6, "num_experts_per_tok": 2, "intermediate_size": 96,
    "intermediate_size_mlp": 160, "vocab_size": 320, "rope_theta": 50000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 2.0, "high_freq_factor": 2.0,
                     "original_max_position_embeddings": 32},
    "use_qk_norm": True, "attention_chunk_size": 80, "no_rope_layers": [1, 0, 1, 1, 0],
    "attn_temperature_tuning": True, "floor_scale": 20.0, "attn_scale": 0.2, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
}


def make_model_dir(path: Path, preset_name: str, seed: int, norm_noise: float = 0.0, dtype=torch.bfloat16, **overrides) -> Path:
    from jax_llm_examples_b200 import preset, write_random_model

    cfg = dict(TINY_C, **overrides) if preset_name == "tiny_c" else preset(preset_name, **overrides)
    return write_random_model(path, cfg, seed, dtype=dtype, norm_noise=norm_noise)


@functools.lru_cache(maxsize=64)
def _plain_model(model_dir: str):
    return plain.load_config(model_dir), plain.load_weights(model_dir, torch.float32)


def moe_layer_indices(model_dir) -> list[int]:
    cfg, _ = _plain_model(str(model_dir))
    return [i for i in range(cfg["num_hidden_layers"]) if plain.layer_is_moe(cfg, i)]


def plain_logits(model_dir, tokens, routing: dict[int, np.ndarray] | None = None, differing: list | None = None
                 ) -> tuple[np.ndarray, float]:
    """Logits [T, V] of the plain implementation in float32.  With ``routing`` ({layer: experts
    [T, k]}) it takes those experts instead of its own choice and also returns by how much, at
    worst, a taken expert's score lay below the score it needed to be chosen (0 = same choice).
    ``differing`` collects [choices that differ from the plain implementation's own, all choices]."""
    cfg, w = _plain_model(str(model_dir))
    stats: dict = {}
    with torch.no_grad():
        out = plain.forward(cfg, w, list(tokens), stats, routing).numpy()
    gaps = list(stats.get("router_shortfall", {}).values())
    worst = max((float(g.max()) for g in gaps), default=0.0)
    if differing is not None:
        differing[0] += sum(int((g > 0).sum()) for g in gaps)
        differing[1] += sum(g.numel() for g in gaps)
    return out, worst


def as_rows_sum(x) -> torch.Tensor:
    """What a part returned, as one tensor: split-K partials are added, a sum of terms is made."""
    if hasattr(x, "materialize"):
        return x.materialize()
    data, splits = (x.data, x.splits) if hasattr(x, "splits") else (x, 1)
    return data.sum(0) if splits > 1 or data.dim() == 3 else data


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    """Largest difference of a row, relative to that row's largest reference logit; max over rows."""
    a, b = np.atleast_2d(a), np.atleast_2d(b)
    return float(np.max(np.max(np.abs(a - b), axis=-1) / np.maximum(np.max(np.abs(b), axis=-1), 1e-6)))


# Tolerances follow the precisions: float32 has eps 6e-8 and a few thousand roundings per logit;
# bfloat16 rounds activations (eps 4e-3) a few times per layer.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def random_requests(rng: random.Random, vocab: int, lengths: list[int]) -> dict[str, list[int]]:
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


# ------------------------------------------------------------------------------------ traces
def trace_whole(requests):
    """Each request alone, whole, in one step."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def trace_tail_decode(requests, tail=32):
    """Most of a request in one step, then its last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(len(toks) - tail, 0)
        if head:
            steps.append({"entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": [rid] if i == len(toks) - 1 else []})
    return steps


def trace_portions(requests, rng: random.Random):
    """Portions of changing size, down to two tokens."""
    steps = []
    sizes = [7, 2, 19, 3, 2, 11, 5, 2, 13, 4]
    for rid, toks in requests.items():
        at, k = 0, rng.randrange(len(sizes))
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            steps.append({"entries": [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}],
                          "end": [rid] if at + n == len(toks) else []})
            at += n
    return steps


SHORT_PORTIONS = (2, 2, 3, 5, 8, 17, 33)
# around the sizes at which the attention part changes kernels (64 tokens) and tiles (128 rows)
LONG_PORTIONS = (2, 17, 63, 64, 65, 127, 128, 129, 200, 300)


def trace_mixed(requests, rng: random.Random, max_live=4, portions=SHORT_PORTIONS):
    """Up to `max_live` live requests: portions of some beside single tokens of others; a request
    may sit out a step; finished requests make room (and pages) for the next ones."""
    pending = list(requests.items())
    live: dict[str, int] = {}
    steps = []
    while pending or live:
        while pending and len(live) < max_live and (not live or rng.random() < 0.7):
            rid, _ = pending.pop(0)
            live[rid] = 0
        entries, end = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            toks, at = requests[rid], live[rid]
            left = len(toks) - at
            if rng.random() < 0.5 or left == 1:
                n = 1
            else:
                n = min(left, rng.choice(portions))
            entries.append({"id": rid, "tokens": toks[at:at + n], "want": list(range(n))})
            live[rid] = at + n
            if live[rid] == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def run_trace(engine, steps):
    """Drives the engine's step function with a trace.  Returns (logits by (request, position),
    expert choices by (request, position): one array [k] per routed layer, in layer order)."""
    from jax_llm_examples_b200 import StepEntry

    engine.record_routing = True
    slots: dict[str, int] = {}
    at: dict[str, int] = {}
    out: dict[tuple[str, int], np.ndarray] = {}
    routing: dict[tuple[str, int], list[np.ndarray]] = {}
    for st in steps:
        entries, places, fed = [], [], []
        for e in st["entries"]:
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.new_request()
                at[rid] = 0
            entries.append(StepEntry(slots[rid], e["tokens"], e["want"]))
            places += [(rid, at[rid] + w) for w in e["want"]]
            fed += [(rid, at[rid] + i) for i in range(len(e["tokens"]))]
            at[rid] += len(e["tokens"])
        logits = engine.step(entries).cpu().numpy()
        engine.check_status()
        # which attention kernels served the step together (a set of tuples, kept on the engine for the tests)
        engine.__dict__.setdefault("attention_kernels_seen", set()).update(engine.last_scratch.get("attention_kernels", ()))
        assert logits.shape[0] == len(places)
        for row, key in zip(logits, places):
            out[key] = row
        choices = [t.cpu().numpy() for t in engine.last_routing]
        for n, key in enumerate(fed):
            routing[key] = [c[n] for c in choices]
        for rid in st["end"]:
            engine.finish(slots.pop(rid))
        engine.manager.check()
    return out, routing


# A router score is a logit of the layer's hidden state, so it carries the error a logit carries, and a choice
# compares two of them.  A difference below this fraction of the layer's typical score (RMS over the sequence)
# is therefore a tie that either precision may break either way: in bfloat16 the bound of a logit (TOL); in
# float32, where sums of D products differ by ~1e-6 relative, half of it.  How many choices fall into that band
# depends on the number of experts (with 40 experts and top-1, 1.1 % were seen; with 4 to 16, under 0.5 %); a
# fault in the routing itself (a wrong expert table, a wrong tie rule) changes tens of percent: the share of
# differing choices is capped well between the two.
TIE = {"float32": 1e-5, "bfloat16": TOL["bfloat16"]}
TIE_SHARE = 0.05


def compare_with_plain(model_dir, requests, got, routing, dtype: str):
    """Every logit row the trace produced against the plain implementation's row at that place.
    The plain implementation takes the engine's experts; they must be its own choice too, except
    where the scores tie."""
    worst = 0.0
    layers = moe_layer_indices(model_dir)
    differing = [0, 0]
    for rid, toks in requests.items():
        forced = None
        if layers:
            forced = {L: np.stack([routing[(rid, p)][j] for p in range(len(toks))]) for j, L in enumerate(layers)}
        ref, shortfall = plain_logits(model_dir, toks, forced, differing)
        assert shortfall < TIE[dtype], f"{dtype}: request {rid}: an expert was chosen whose score is too low by {shortfall:.2e} of the layer's typical score"
        for pos in range(len(toks)):
            if (rid, pos) not in got:
                continue
            err = rel_err(got[(rid, pos)], ref[pos])
            assert err < TOL[dtype], f"{dtype}: request {rid} position {pos}: relative error {err:.3e}"
            worst = max(worst, err)
    assert differing[0] <= TIE_SHARE * differing[1], f"{dtype}: {differing[0]} of {differing[1]} expert choices differ"
    return worst


def compare_plain_only(model_dir, requests, got, dtype: str):
    """As compare_with_plain, with the plain implementation's own expert choices."""
    for rid, toks in requests.items():
        ref, _ = plain_logits(model_dir, toks)
        for pos in range(len(toks)):
            if (rid, pos) in got:
                err = rel_err(got[(rid, pos)], ref[pos])
                assert err < TOL[dtype], f"{dtype}: request {rid} position {pos}: relative error {err:.3e}"


def plain_greedy_checked(folder, prompt, got, dtype: str):
    """`got` must be the plain implementation's greedy continuation, except that a step whose two best
    logits nearly tie (closer than the precision can tell apart) may go either way; after such a step the
    comparison follows the engine's choice."""
    cfg, w = _plain_model(str(folder))
    toks = list(prompt)
    tol = 1e-5 if dtype == "float32" else 2e-2
    with torch.no_grad():
        for step, g in enumerate(got):
            logits = plain.forward(cfg, w, toks)[-1]
            best = int(torch.argmax(logits))
            if g != best:
                gap = float(logits[best] - logits[g]) / float(logits.abs().max())
                assert gap < tol, f"{dtype}: step {step}: engine chose {g}, plain {best}, relative logit gap {gap:.2e}"
            toks.append(g)
