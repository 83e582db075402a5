"""Benchmark of the engine on one B200: decode tokens/s at batch 8 and context 8192 on Scout-sized
layers with random weights (the headline), the same end to end through the Python entry point,
a 2,048-token prefill, decode at batch 1 and 64, and the decode step's share of the HBM roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

One JSON line on stdout.  A "step" is one decode step of the whole batch.  Random weights
N(0, 0.02) and seeded uniform token ids; the cache of the timed requests is filled with random
keys and values up to the context length instead of being computed by a prefill of batch x 8192
tokens (what a decode step reads and computes does not depend on the values).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_SCOUT_B1 = 85.5  # tok/s, TPU v5e-16, int8, 48 layers (llama4/README.md:73-75): not comparable, recorded only


def _peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"])}, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self):
        self.rows: list[list[str]] = []
        self.proc = None

    @staticmethod
    def _device_id() -> str:
        """The running device as nvidia-smi knows it: its UUID (index 0 of this process may be another index there)."""
        try:
            import torch

            return "GPU-" + str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
        except Exception:
            return "0"

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self._device_id(), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [r for r in self.rows if len(r) == 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "reasons": reasons, "samples": len(rows),
                "power_w_max": max(float(r[2]) for r in rows if r[2].replace(".", "").isdigit())}


def _fill_cache(engine, slots, length, gen):
    """Gives each slot `length` tokens of random keys and values (reserve + commit, no model run)."""
    import torch

    for s in slots:
        engine.manager.reserve(s, length)
        engine.manager.commit(s, length)
    for t in engine.kv:
        flat = t.view(-1)
        step = 1 << 28
        for lo in range(0, flat.numel(), step):
            hi = min(flat.numel(), lo + step)
            flat[lo:hi] = (0.5 * torch.randn(hi - lo, generator=gen, device=t.device, dtype=torch.float32)).to(t.dtype)


def _decode_bytes(model, engine, batch, ctx_len, routing) -> float:
    """Bytes a decode step has to read: every weight it uses once (attention, shared expert, router,
    the DISTINCT routed experts of each layer, norms, the LM head) and the cache of the live requests."""
    import torch

    from jax_llm_examples_b200.parts import RoutedExperts

    total = model.lm_head.numel() * model.lm_head.element_size()
    total += batch * model.hidden_size * model.embedding.element_size()
    moe_i = 0
    for blk in model.blocks:
        m, f = blk.mixer, blk.feed_forward
        total += sum(w.numel() * w.element_size() for w in (m.w_qkv, m.w_o))
        if isinstance(f, RoutedExperts):
            distinct = int(torch.unique(routing[moe_i]).numel())
            moe_i += 1
            per_expert = (f.we_gate_up[0].numel() + f.we_down[0].numel()) * f.we_gate_up.element_size()
            total += distinct * per_expert + f.w_router.numel() * 4
            total += sum(w.numel() * w.element_size() for w in (f.shared.w_gate_up, f.shared.w_down))
        else:
            total += sum(w.numel() * w.element_size() for w in (f.w_gate_up, f.w_down))
    for need in model.plan.caches:
        keys = ctx_len if need.retention.kind == 0 else min(ctx_len, (ctx_len % need.retention.size) or need.retention.size)
        total += batch * keys * 2 * need.num_kv_heads * need.head_dim * engine.kv[0].element_size()
    return float(total)


def _prefill_flops(cfg, tokens: int) -> float:
    D, Hq, Hkv, dh = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    per_layer = 0.0
    total = 0.0
    for i in range(cfg.num_hidden_layers):
        lin = 2 * tokens * D * (Hq + 2 * Hkv) * dh + 2 * tokens * Hq * dh * D
        attn = 4 * Hq * dh * tokens * (tokens + 1) / 2
        if cfg.layer_is_moe(i):
            F = cfg.intermediate_size
            ffn = 2 * tokens * 3 * D * F * (cfg.num_experts_per_tok + 1) + 2 * tokens * D * cfg.num_local_experts
        else:
            ffn = 2 * tokens * 3 * D * cfg.intermediate_size_mlp
        total += lin + attn + ffn
    return total + 2 * D * cfg.vocab_size


def run_ours(args) -> dict:
    import torch

    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.kernels import api

    peaks, peak_src = _peaks()
    torch.cuda.set_device(0)
    cfg_json = J.preset(args.preset, num_hidden_layers=args.layers) if args.layers else J.preset(args.preset)
    full_layers = J.preset(args.preset)["num_hidden_layers"]
    ctx_len, batch, page = args.context, args.batch, 64
    t0 = time.time()
    model = J.random_model(cfg_json, seed=0, dtype="bfloat16")
    cfg = model.config
    torch.cuda.synchronize()
    print(f"[bench] model of {cfg.num_hidden_layers} layers ({model.weight_bytes() / 1e9:.1f} GB) made in {time.time() - t0:.0f} s", file=sys.stderr)
    known = {"wide", "past_chunk", "ref_table", "prefill4", "long"}
    extra = set() if args.extra_points == "none" or args.skip_points else (
        set(known) if args.extra_points == "all" else set(filter(None, args.extra_points.split(","))))
    if extra - known:
        raise SystemExit(f"bench.py: unknown --extra-points {sorted(extra - known)}; known: {sorted(known)}")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    import random as pyrandom

    rng = pyrandom.Random(0)

    def decode_run(b: int, steps: int, warmup: int, e2e: bool = False, ctx_len: int = ctx_len, start_len: int | None = None,
                   max_seq_len: int | None = None):
        """b requests decode steps + warmup tokens; they end just below ctx_len tokens, or start at start_len.
        ``max_seq_len``: the longest request the engine allows (default: ctx_len)."""
        g = J.Generator(model, max_tokens=b * ctx_len, page_size=page, max_slots=b, max_tokens_per_step=max(b, 2048),
                        max_seq_len=max_seq_len or ctx_len)
        eng = g.engine
        slots = [eng.new_request() for _ in range(b)]
        if start_len is None:
            start_len = ctx_len - (steps + warmup) - 10
        _fill_cache(eng, slots, start_len, gen)
        extra_steps = 8  # untimed steps after the timed ones, to see which experts a step touches
        # fresh token ids for every step (drawn beforehand), so that every step routes its own way
        all_toks = [[rng.randrange(cfg.vocab_size) for _ in range(b)] for _ in range(steps + warmup + extra_steps)]
        out_host = torch.empty(b, dtype=torch.int32).pin_memory()
        sampler = J.Sampler(0)
        at = [0]

        def one_step():
            entries = [J.StepEntry(s, [t], [0]) for s, t in zip(slots, all_toks[at[0]])]
            at[0] += 1
            logits = eng.step(entries)
            nxt = sampler.sample(logits, [0.0] * b, [0] * b, [0] * b, [0] * b)
            out_host.copy_(nxt, non_blocking=True)
            return nxt

        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        launches0 = api.launch_count() + eng.graph_kernel_launches
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_host = time.perf_counter()
        ev0.record()
        for _ in range(steps):
            one_step()
        ev1.record()
        torch.cuda.synchronize()
        host_ms = (time.perf_counter() - t_host) * 1e3
        dev_ms = ev0.elapsed_time(ev1)
        eng.check_status()
        launches = api.launch_count() + eng.graph_kernel_launches - launches0
        # which experts a step touches: a few more steps, untimed, with the choices recorded; the bytes of a step
        # are the mean over them (the cache that a timed step reads: the requests' mean length over the timed steps)
        eng.record_routing = True
        nbytes = 0.0
        for _ in range(extra_steps):
            one_step()
            torch.cuda.synchronize()
            nbytes += _decode_bytes(model, eng, b, start_len + warmup + (steps + 1) // 2, eng.last_routing) / extra_steps
        desc_bytes = 4 * J.CacheManager.packed_size(len(eng.manager.groups), b, b, b, -(-ctx_len // page))
        for s in slots:
            eng.finish(s)
        del g, eng
        torch.cuda.empty_cache()
        return {"ms": (host_ms if e2e else dev_ms) / steps, "bytes": nbytes, "launches": launches, "h2d": desc_bytes, "d2h": 4 * b}

    def e2e_run(b: int, steps: int, warmup: int):
        """The same decode steps through the public entry point (Generator: scheduler, step function,
        sampler): each step packs host token ids, copies them to the device, and reads the sampled
        ids back to the host, where the scheduler appends them to the requests."""
        g = J.Generator(model, max_tokens=b * ctx_len, page_size=page, max_slots=b, max_tokens_per_step=max(b, 2048),
                        max_seq_len=ctx_len)
        eng, sch = g.engine, g.scheduler
        start_len = ctx_len - (steps + warmup) - 2
        reqs = []
        for i in range(b):
            r = J.Request(i, [rng.randrange(cfg.vocab_size) for _ in range(start_len + 1)],
                          J.SamplingParams(max_new_tokens=steps + warmup + 8))
            r.slot = eng.new_request()
            r.fed = start_len  # everything but the prompt's last token is "in the cache" (random contents)
            sch.running.append(r)
            reqs.append(r)
        _fill_cache(eng, [r.slot for r in reqs], start_len, gen)
        for _ in range(warmup):
            sch.step()
        torch.cuda.synchronize()
        h0, d0 = g.h2d_bytes, g.d2h_bytes
        t_host = time.perf_counter()
        for _ in range(steps):
            sch.step()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t_host) * 1e3 / steps
        assert all(len(r.output) == steps + warmup for r in reqs)
        desc = 4 * J.CacheManager.packed_size(len(eng.manager.groups), b, b, b, -(-ctx_len // page))
        for r in reqs:
            if r.slot is not None:
                eng.finish(r.slot)
        return {"ms": ms, "h2d": desc, "d2h": (g.d2h_bytes - d0) // steps}

    points = {}
    # The order of the measurements follows what each is sensitive to.  The prompt measurements run the library's dense
    # products, whose rate goes with the power the GPU may draw: they come first, while it is cool, as the peak they are
    # set against was measured (a burst).  Then the headline: the decode steps, with the clocks sampled.  Decoding at
    # batch 1 is a chain of short kernels and goes with the SM clock: it is the first of the further points.  The
    # decode points at larger batches are bound by HBM and mind neither: they come last.
    # prefill of one 2,048-token prompt
    T = args.prefill_tokens
    g = J.Generator(model, max_tokens=T + page, page_size=page, max_slots=1, max_tokens_per_step=T)
    eng = g.engine
    prompt = [rng.randrange(cfg.vocab_size) for _ in range(T)]
    pre_ms = []
    for it in range(0 if args.skip_prefill else 3 + 3):
        s = eng.new_request()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        eng.step([J.StepEntry(s, prompt, [T - 1])])
        ev1.record()
        torch.cuda.synchronize()
        if it >= 3:
            pre_ms.append(ev0.elapsed_time(ev1))
        eng.finish(s)
    pre = sorted(pre_ms)[len(pre_ms) // 2] if pre_ms else float("nan")
    flops = _prefill_flops(cfg, T)
    del g, eng
    torch.cuda.empty_cache()

    # a mixed step: the batch's decoded tokens beside one T-token prompt portion, in one step
    if not args.skip_points and not args.skip_prefill:
        g = J.Generator(model, max_tokens=batch * ctx_len + T + page, page_size=page, max_slots=batch + 1,
                        max_tokens_per_step=T + batch, max_seq_len=ctx_len)
        eng = g.engine
        slots = [eng.new_request() for _ in range(batch)]
        _fill_cache(eng, slots, ctx_len - 16, gen)
        mixed_ms = []
        for it in range(3 + 3):
            s = eng.new_request()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            eng.step([J.StepEntry(x, [rng.randrange(cfg.vocab_size)], [0]) for x in slots] + [J.StepEntry(s, prompt, [T - 1])])
            ev1.record()
            torch.cuda.synchronize()
            if it >= 3:
                mixed_ms.append(ev0.elapsed_time(ev1))
            eng.finish(s)
        eng.check_status()
        points[f"mixed_b{batch}_plus_{T}_ms"] = round(sorted(mixed_ms)[len(mixed_ms) // 2], 3)
        del g, eng
        torch.cuda.empty_cache()

    clocks = ClockSampler()
    clocks.start()
    main = decode_run(batch, args.steps, args.warmup, e2e=False)
    clock_rec = clocks.stop()
    e2e = e2e_run(batch, args.steps, args.warmup) if not args.skip_e2e else {"ms": float("nan"), "h2d": 0, "d2h": 0}

    few = max(3, min(args.steps, 20))

    def point(name: str, b: int, **kw):
        r = decode_run(b, few, 3, **kw)
        points[name] = round(b / (r["ms"] / 1e3), 1)
        points[name + "_hbm_frac"] = round(r["bytes"] / (r["ms"] / 1e3) / 1e9 / peaks["hbm_gbs"], 3)

    if not args.skip_points:
        point("decode_b1", 1)
    if not args.skip_points:
        point("decode_b64", 64)
    if "wide" in extra:
        # the same decode steps on an engine that allows requests of 131072 tokens (the default when the pool is
        # sized from free memory): the captured graphs are planned for the context in use, not for the widest request
        point(f"decode_b{batch}_max_seq_131072", batch, max_seq_len=131072)
    if "past_chunk" in extra and cfg.attention_chunk_size:
        # just past a chunk start the rotary layers read almost no cache; only the NoPE layers read the history
        C = cfg.attention_chunk_size
        point(f"decode_b{batch}_just_past_{C}", batch, ctx_len=C + 512, start_len=C + 16)
    if "ref_table" in extra:
        # the settings of the reference's published table (llama4/README.md:73-77): context 4096, batch 1, 16, 32
        for b in (1, 16, 32):
            point(f"decode_b{b}_ctx4096", b, ctx_len=4096)

    if "prefill4" in extra:
        # four 2048-token prompts in one step: the routed experts get four times the rows each
        g = J.Generator(model, max_tokens=4 * (T + page), page_size=page, max_slots=4, max_tokens_per_step=4 * T)
        eng, ms = g.engine, []
        for it in range(3 + 3):
            ss = [eng.new_request() for _ in range(4)]
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            eng.step([J.StepEntry(x, [rng.randrange(cfg.vocab_size) for _ in range(T)], [T - 1]) for x in ss])
            ev1.record()
            torch.cuda.synchronize()
            if it >= 3:
                ms.append(ev0.elapsed_time(ev1))
            for x in ss:
                eng.finish(x)
        eng.check_status()
        m = sorted(ms)[len(ms) // 2]
        points[f"prefill_4x{T}_tok_s"] = round(4 * T / (m / 1e3), 1)
        points[f"prefill_4x{T}_ms"] = round(m, 3)
        del g, eng
        torch.cuda.empty_cache()
    if "long" in extra:
        # one long prompt in portions of T tokens (chunk starts crossed, pages of dead chunks given back), then 256
        # decoded tokens; device-timed
        L, n_dec = args.long_tokens, 256
        g = J.Generator(model, max_tokens=L + n_dec + page, page_size=page, max_slots=1, max_tokens_per_step=T)
        eng = g.engine
        s = eng.new_request()
        toks = [rng.randrange(cfg.vocab_size) for _ in range(L + n_dec)]
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
        for a in range(0, L, T):
            eng.step([J.StepEntry(s, toks[a:a + T], [T - 1] if a + T >= L else [])])
        ev[1].record()
        n_warm = 3  # the first decode steps run eagerly and capture the graph that the others replay: not timed
        for i in range(n_dec):
            if i == n_warm:
                ev[2].record()
            eng.step([J.StepEntry(s, [toks[L + i]], [0])])
        ev[3].record()
        torch.cuda.synchronize()
        eng.check_status()
        points[f"long_{L}_prefill_tok_s"] = round(L / (ev[0].elapsed_time(ev[1]) / 1e3), 1)
        points[f"long_{L}_decode_b1_tok_s"] = round((n_dec - n_warm) / (ev[2].elapsed_time(ev[3]) / 1e3), 1)
        eng.finish(s)
        del g, eng
        torch.cuda.empty_cache()

    tok_s = batch / (main["ms"] / 1e3)
    achieved = main["bytes"] / (main["ms"] / 1e3) / 1e9
    return {
        "metric": f"decode tok/s at batch {batch}, context {ctx_len} (Llama 4 {'Scout' if args.preset == 'scout16' else args.preset} layer sizes)",
        "value": round(tok_s, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms"], 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights, seeded uniform token ids (fresh ones every step), random cache contents",
        "config": {
            "model": "llama4-scout-layer-sizes" if args.preset == "scout16" else f"llama4-{args.preset}", "layers": cfg.num_hidden_layers, "layers_full_config": full_layers,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "experts": cfg.num_local_experts, "top_k": cfg.num_experts_per_tok,
            "expert_inter": cfg.intermediate_size, "vocab": cfg.vocab_size, "chunk": cfg.attention_chunk_size,
            "global_batch": batch, "seq_len": ctx_len, "page_size": page, "parallelism": "none (1 GPU)",
            "l2": "inputs larger than L2: each step reads its weights (GBs) once", "peaks": peak_src,
        },
        "e2e": {"value": round(batch / (e2e["ms"] / 1e3), 1), "unit": "tok/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": main["launches"],
        "clocks": clock_rec,
        "prefill": {"value": round(T / (pre / 1e3), 1), "tokens": T, "ms": round(pre, 3),
                    "frac": round(flops / (pre / 1e3) / 1e12 / peaks["bf16_tflops"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "published_not_comparable": {"scout_b1_tpu_v5e16_int8_tok_s": PUBLISHED_SCOUT_B1},
    }


def run_reference(args) -> dict:
    """The reference arm: the UNMODIFIED reference installed under baseline/_ref, through its own public calls
    (``prefill`` then ``decode_step`` over a fixed batch, llama4/llama4_jax/model.py:1243-1277, the loop of
    llama4/main.py:68-75), at the same layer sizes, batch and context, with its own random initialisation
    (``Weights.init``) and its cache in bfloat16.  Nothing of this repository's engine is on that path.  Where the
    reference cannot be imported or run here, the line says why, with the exception it raised."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "llama4_jax")):
        return {"impl": "reference", "unavailable": f"the reference is not installed under {os.path.relpath(ref_root, ROOT)}"}
    sys.path.insert(0, ref_root)
    try:
        import dataclasses

        import jax
        import jax.numpy as jnp
        import numpy as np
        from jax import random
        from jax.sharding import AxisType
        from llama4_jax import model as l4jax
    except Exception as e:  # on this image: No module named 'jax' (not in the image, not in the offline wheelhouse)
        return {"impl": "reference", "unavailable": f"import of llama4_jax from baseline/_ref failed: {type(e).__name__}: {e}"}
    try:
        import jax_llm_examples_b200 as J

        text = J.preset(args.preset, num_hidden_layers=args.layers) if args.layers else J.preset(args.preset)
        batch, ctx_len, steps, warmup = args.batch, args.context, args.steps, max(args.warmup, 3)
        mesh = jax.make_mesh((1, 1, 1), ("x", "y", "z"), devices=jax.devices()[:1], axis_types=(AxisType.Explicit,) * 3)
        cfg = l4jax.hf_to_jax_config(text)
        cfg = dataclasses.replace(cfg, mesh=mesh, max_seq_len=ctx_len, quant_attn=False, quant_moe=False, quant_mlp=False,
                                  quant_cache=False)
        with jax.sharding.set_mesh(cfg.mesh):
            weights = l4jax.Weights.init(random.key(0), cfg)
            cache = l4jax.KVCache.init(random.key(1), cfg, batch, cfg.max_seq_len)
            prompt = np.random.default_rng(0).integers(1, cfg.vocab_size, size=(batch, ctx_len - steps - warmup - 2))
            next_tokens, _, cache = l4jax.prefill(jnp.asarray(prompt, dtype=jnp.int32), weights, cache, cfg)
            cur = next_tokens[:, cache.iter - 1: cache.iter]
            for _ in range(warmup):
                cur, cache = l4jax.decode_step(cur, weights, cache, cfg)
            np.asarray(cur)
            t0 = time.perf_counter()
            for _ in range(steps):
                cur, cache = l4jax.decode_step(cur, weights, cache, cfg)
                np.asarray(cur)  # the step's tokens on the host, as the reference's loop collects them
            ms = (time.perf_counter() - t0) * 1e3 / steps
        value = round(batch / (ms / 1e3), 1)
        return {"impl": "reference", "metric": f"decode tok/s at batch {batch}, context {ctx_len}", "value": value, "unit": "tok/s",
                "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 3), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic: the reference's own random weights, uniform token ids",
                "config": {"model": args.preset, "layers": cfg.num_layers, "global_batch": batch, "seq_len": ctx_len, "parallelism": "none (1 GPU)"},
                "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4 * batch}}
    except Exception as e:
        return {"impl": "reference", "unavailable": f"the reference was imported but did not run: {type(e).__name__}: {str(e)[:300]}"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="scout16", help="named configuration (the default is the benchmark's: 16 Scout-sized layers)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (same layer sizes)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--extra-points", default="all", help="'all' (the default), 'none', or a comma list of further points: wide (an engine that allows 131072-token "
                    "requests), past_chunk (decode just past a chunk start), ref_table (context 4096, batch 1/16/32), "
                    "prefill4 (four prompts in one step), long (one --long-tokens prompt in portions, then 256 decoded tokens)")
    ap.add_argument("--long-tokens", type=int, default=32768)
    ap.add_argument("--skip-e2e", action="store_true", help="skip the end-to-end run (for profiling captures)")
    ap.add_argument("--skip-prefill", action="store_true", help="skip the prefill measurement (for profiling captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps(run_reference(args)))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
