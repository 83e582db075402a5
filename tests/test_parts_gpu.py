"""The parts of the decoder alone, and the generality of their arrangement: a toy architecture defined HERE
(a mixer with per-request state of its own, a feed-forward with softmax routing, a half-split rotary
encoding) is registered, loaded from a model folder and stepped through the engine without any change to
the package; and schedules that run a block twice or let a layer read another layer's cache."""

import dataclasses
import json
import math
import random

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.plain import llama4_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"


# ------------------------------------------------------------------------------- parts alone
def _ctx(J, runtime, q_lens, starts, page_size=16, n_pages=32, vocab=100):
    """A step context for hand-made batches (what Engine.step builds), with one block table."""
    from jax_llm_examples_b200.parts import StepContext, Workspace, plan_attention_tiles

    pos = [s + i for n, s in zip(q_lens, starts) for i in range(n)]
    req = [r for r, n in enumerate(q_lens) for _ in range(n)]
    t = lambda v: torch.tensor(v, device=DEV, dtype=torch.int32)
    width = max(-(-(s + n) // page_size) for n, s in zip(q_lens, starts))
    perm = torch.randperm(n_pages)[: len(q_lens) * width].reshape(len(q_lens), width).to(torch.int32).to(DEV)
    N = sum(q_lens)
    ctx = StepContext(runtime=runtime, n_tokens=N, n_requests=len(q_lens), token_ids=t([0] * N), positions=t(pos),
                      req_of_token=t(req), cu_q=t(list(np.concatenate([[0], np.cumsum(q_lens)]))), q_start=t(starts),
                      kv_len=t([s + n for n, s in zip(q_lens, starts)]), slot_ids=t(list(range(len(q_lens)))),
                      logit_rows=t([]), n_logit_rows=0, status=torch.zeros(1, device=DEV, dtype=torch.int32),
                      host_q_lens=list(q_lens), host_q_start=list(starts), host_slot_ids=list(range(len(q_lens))),
                      max_q_len=max(q_lens), max_kv_len=max(s + n for n, s in zip(q_lens, starts)),
                      workspace=Workspace(torch.device(DEV)))
    ctx.plan_with((plan_attention_tiles,), page_size)
    return ctx, perm


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
def test_norm_part(dtype, tol):
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.parts import RMSNorm, Runtime

    rt = Runtime(dtype, torch.device(DEV))
    ctx, _ = _ctx(J, rt, [7], [0])
    g = 1 + 0.1 * torch.randn(200, device=DEV)
    x, d = torch.randn(7, 200, device=DEV), torch.randn(7, 200, device=DEV)
    h, h32, routing = RMSNorm(g, 1e-6).forward(ctx, x.clone(), d, out_dtype=dtype, want_f32=True)
    ref = plain.rms_norm((x + d).cpu(), g.cpu(), 1e-6)
    assert routing is None and H.rel_err(h.float().cpu().numpy(), ref.numpy()) < tol
    assert H.rel_err(h32.cpu().numpy(), ref.numpy()) < 3e-6


@pytest.mark.parametrize("k, splits", [(2, 3), (16, 5)])
def test_norm_part_adds_an_expert_layers_rows_in_the_kernel_or_lets_their_producer(k, splits):
    """A sum of terms (rows still in expert order) is added by the norm's kernel as long as a token adds no more rows and
    partials than the kernel takes (64); beyond that the norm asks the producer for the finished sum."""
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.kernels import api as K
    from jax_llm_examples_b200.parts import RMSNorm, Rows, RowSum, Runtime

    N, D = 5, 1024
    rt = Runtime(torch.bfloat16, torch.device(DEV))
    ctx, _ = _ctx(J, rt, [N], [0])
    g = 1 + 0.1 * torch.randn(D, device=DEV)
    x, y = torch.randn(N, D, device=DEV), torch.randn(splits, N * k, D, device=DEV)
    pos = torch.randperm(N * k, device=DEV).to(torch.int32)
    total = y.sum(0)[pos.long()].reshape(N, k, D).sum(1)
    asked = []

    def materialize():
        asked.append(True)
        return total.clone()

    h, _, _ = RMSNorm(g, 1e-6).forward(ctx, x.clone(), RowSum([Rows(y, splits, pos, k, 0)], materialize), out_dtype=torch.bfloat16)
    ref = plain.rms_norm((x + total).cpu(), g.cpu(), 1e-6)
    assert H.rel_err(h.float().cpu().numpy(), ref.numpy()) < 1e-2
    assert bool(asked) == (k * splits > K.DELTA_MAX_STREAMS)


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("rope, chunk, dh", [(True, 24, 32), (False, None, 64)])
def test_attention_part_with_its_position_encoding(dtype, tol, rope, chunk, dh):
    """PagedAttention + position encoding alone: a prompt portion after cached tokens, and a decode token."""
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.parts import (InterleavedRope, LayerCache, NoPositionWithTemperature, PagedAttention, Runtime,
                                             llama3_scaled_frequencies)

    torch.manual_seed(0)
    rt = Runtime(dtype, torch.device(DEV))
    D, Hq, Hkv, eps = 96, 4, 2, 1e-5
    wq, wk, wv = (torch.randn(n, D) * 0.1 for n in (Hq * dh, Hkv * dh, Hkv * dh))
    wo = torch.randn(D, Hq * dh) * 0.1
    cfg = {"head_dim": dh, "rope_theta": 10000.0, "rope_scaling": None}
    pos_part = InterleavedRope(llama3_scaled_frequencies(dh, 10000.0, None), DEV) if rope else NoPositionWithTemperature(0.1, 8.0)
    mixer = PagedAttention(torch.cat([wq, wk, wv]).to(dtype).to(DEV), wo.to(dtype).to(DEV), Hq, Hkv, dh, pos_part,
                           qk_norm_eps=eps if rope else None, chunk=chunk)
    T = 60
    hs = torch.randn(T, D)
    pages = torch.zeros(32, 2, Hkv, 16, dh, device=DEV, dtype=dtype)
    outs = []
    table = torch.randperm(32)[:4].reshape(1, 4).to(torch.int32).to(DEV)  # 4 pages of 16 hold the 60 tokens
    for lo, hi in ((0, 37), (37, 59), (59, 60)):  # two portions, then a single token
        ctx, _ = _ctx(J, rt, [hi - lo], [lo])
        out = mixer.forward(ctx, hs[lo:hi].to(dtype).to(DEV), LayerCache(pages, table, True, None))
        outs.append(H.as_rows_sum(out))
        assert int(ctx.status) == 0
    got = torch.cat(outs).cpu()
    # plain: whole sequence
    w = lambda m: m.to(dtype).float()
    h = hs.to(dtype).float()
    positions = torch.arange(T)
    q, k, v = (h @ w(wq).T).reshape(T, Hq, dh), (h @ w(wk).T).reshape(T, Hkv, dh), (h @ w(wv).T).reshape(T, Hkv, dh)
    if rope:
        f = plain.rope_inverse_frequencies(cfg)
        q, k = plain.apply_rope_interleaved(q, positions, f), plain.apply_rope_interleaved(k, positions, f)
        q, k = plain.rms_norm(q, None, eps), plain.rms_norm(k, None, eps)
    else:
        q = q * plain.attention_temperature(positions, 8.0, 0.1)[:, None, None]
    a = plain.gqa_attention(q, k, v, plain.attention_mask(positions, chunk))
    ref = a.reshape(T, -1) @ w(wo).T
    assert H.rel_err(got.numpy(), ref.numpy()) < tol


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
def test_feed_forward_parts(dtype, tol):
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.parts import DenseSwiGLU, RoutedExperts, Runtime

    torch.manual_seed(1)
    rt = Runtime(dtype, torch.device(DEV))
    N, D, F, E, k = 23, 72, 48, 5, 2
    ctx, _ = _ctx(J, rt, [N], [0])
    r = lambda *s: (torch.randn(*s) * 0.2).to(dtype)
    wg, wu, wd = r(F, D), r(F, D), r(D, F)
    h32 = torch.randn(N, D)
    dense = DenseSwiGLU(torch.cat([wg, wu]).to(DEV), wd.to(DEV))
    got = H.as_rows_sum(dense.forward(ctx, h32.to(dtype).to(DEV), None)).cpu()
    hq = h32.to(dtype).float()
    ref = plain.swiglu(hq, wg.float().T, wu.float().T, wd.float().T)
    assert H.rel_err(got.numpy(), ref.numpy()) < tol
    # routed experts with a shared expert; weights in the checkpoint's orientations
    wr, egu, edn = torch.randn(E, D) * 0.3, r(E, D, 2 * F), r(E, F, D)
    shared = DenseSwiGLU(torch.cat([wg, wu]).to(DEV), wd.to(DEV))
    moe = RoutedExperts(wr.to(DEV), egu.transpose(1, 2).contiguous().to(DEV), edn.transpose(1, 2).contiguous().to(DEV), k, shared)
    ctx.scratch["record_routing"] = []
    got = H.as_rows_sum(moe.forward(ctx, h32.to(dtype).to(DEV), h32.to(DEV))).cpu()
    forced = ctx.scratch["record_routing"][0].cpu()
    # the plain MoE takes the unrounded rows (as the engine's router and scaled gather do)
    ref, shortfall = plain.moe(h32, wr.T, egu.float(), edn.float(), wg.float().T, wu.float().T, wd.float().T, k, forced)
    assert float(shortfall.max()) < H.TIE['float32' if dtype == torch.float32 else 'bfloat16']
    assert H.rel_err(got.numpy(), ref.numpy()) < tol
    assert int(ctx.status) == 0


# ------------------------------------------------------------- a toy architecture, defined here
def _register_toy():
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.config import Architecture, read_key
    from jax_llm_examples_b200.parts import (DecoderModel, DenseSwiGLU, FeedForward, Mixer, PagedAttention, PreNormBlock,
                                             RMSNorm, StateNeed, UnfusedEncoding, register_part)
    from jax_llm_examples_b200.weights import TensorSpec

    class DecayStateMixer(Mixer):
        """y_t = s_t with s_t = decay * s_{t-1} + W h_t: a recurrent mixer whose only memory is a state of
        fixed size per request (no keys, no values, no pages)."""

        def __init__(self, w, decay):
            self.w, self.decay = w.float(), float(decay)

        def state_need(self):
            return StateNeed((self.w.shape[0],), torch.float32)

        def forward(self, ctx, h, cache):
            u = h.float() @ self.w.T
            out = torch.empty_like(u)
            at = 0
            for n, slot in zip(ctx.host_q_lens, ctx.host_slot_ids):
                s = cache.state[slot]
                for i in range(n):
                    s = self.decay * s + u[at + i]
                    out[at + i] = s
                cache.state[slot] = s
                at += n
            return out

    class SoftmaxTop1(FeedForward):
        """Softmax over all experts, top-1, the OUTPUT scaled by the probability, no shared expert."""

        def __init__(self, w_router, experts):
            self.w_router, self.experts = w_router.float(), experts

        def forward(self, ctx, h, h32, routing=None):
            p = torch.softmax(h.float() @ self.w_router.T, -1)
            best = p.argmax(-1)
            out = torch.zeros(h.shape[0], h.shape[1], device=h.device)
            for e, ff in enumerate(self.experts):
                rows = torch.nonzero(best == e).flatten()
                if rows.numel():
                    y = ff.forward(ctx, h[rows].contiguous(), None)
                    out[rows] = H.as_rows_sum(y) * p[rows, e][:, None]
            return out

    class HalfSplitRope(UnfusedEncoding):
        """Rotates (x[j], x[j + dh/2]) instead of adjacent pairs."""

        def __init__(self, dh, theta, device):
            self.f = (1.0 / theta ** (torch.arange(0, dh, 2).float() / dh)).to(device)

        def transform(self, ctx, q, k, qk_norm_eps):
            ang = ctx.positions.float()[:, None] * self.f[None]
            s, c = torch.sin(ang)[:, None], torch.cos(ang)[:, None]

            def rot(x):
                x = x.float()
                a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
                return torch.cat([a * c - b * s, b * c + a * s], -1)

            return rot(q), rot(k)

    register_part("mixer", "decay_state", DecayStateMixer)
    register_part("feed_forward", "softmax_top1", SoftmaxTop1)
    register_part("position", "half_split_rope", HalfSplitRope)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        vocab_size: int
        width: int
        layers: int
        heads: int
        head_dim: int
        ffn: int
        experts: int
        decay: float
        eps: float
        window: int

    def parse(d):
        return ToyConfig(*(read_key(d, k, t) for k, t in (("vocab_size", int), ("width", int), ("layers", int), ("heads", int),
                                                           ("head_dim", int), ("ffn", int), ("experts", int),
                                                           ("decay", float), ("eps", float), ("window", int))))

    def specs(c):
        out = [TensorSpec("embed", (c.vocab_size, c.width)), TensorSpec("head", (c.vocab_size, c.width)),
               TensorSpec("norm", (c.width,), "norm")]
        for i in range(c.layers):
            p = f"l{i}."
            out += [TensorSpec(p + "n1", (c.width,), "norm"), TensorSpec(p + "n2", (c.width,), "norm")]
            if i % 2 == 0:
                out += [TensorSpec(p + "state_w", (c.width, c.width))]
                out += [TensorSpec(p + "gu", (2 * c.ffn, c.width)), TensorSpec(p + "down", (c.width, c.ffn))]
            else:
                out += [TensorSpec(p + "qkv", (3 * c.heads * c.head_dim, c.width)), TensorSpec(p + "o", (c.width, c.heads * c.head_dim))]
                out += [TensorSpec(p + "router", (c.experts, c.width))]
                for e in range(c.experts):
                    out += [TensorSpec(p + f"e{e}.gu", (2 * c.ffn, c.width)), TensorSpec(p + f"e{e}.down", (c.width, c.ffn))]
        return {s.name: s for s in out}

    def build(c, t, rt):
        dev = rt.device
        g = lambda n: t.pop(n).to(dev)
        blocks = []
        for i in range(c.layers):
            p = f"l{i}."
            if i % 2 == 0:
                mixer = DecayStateMixer(g(p + "state_w"), c.decay)
                ffn = DenseSwiGLU(g(p + "gu").contiguous(), g(p + "down").contiguous())
            else:
                mixer = PagedAttention(g(p + "qkv").contiguous(), g(p + "o").contiguous(), c.heads, c.heads, c.head_dim,
                                       HalfSplitRope(c.head_dim, 10000.0, dev), window=c.window)
                ffn = SoftmaxTop1(g(p + "router"), [DenseSwiGLU(g(p + f"e{e}.gu").contiguous(), g(p + f"e{e}.down").contiguous())
                                                   for e in range(c.experts)])
            blocks.append(PreNormBlock(RMSNorm(g(p + "n1"), c.eps), mixer, RMSNorm(g(p + "n2"), c.eps), ffn))
        return DecoderModel(rt, g("embed").contiguous(), blocks, RMSNorm(g("norm"), c.eps), g("head").contiguous(), config=c)

    J.register_architecture(Architecture("ToyStateForCausalLM", parse, specs, build))
    return J


TOY = {"architectures": ["ToyStateForCausalLM"], "vocab_size": 90, "width": 40, "layers": 4, "heads": 2, "head_dim": 24,
       "ffn": 48, "experts": 3, "decay": 0.8, "eps": 1e-5, "window": 20}


def _toy_plain(w, c, toks):
    """The toy model on a whole sequence, plain torch float32 on the CPU."""
    T = len(toks)
    x = w["embed"][toks]
    pos = torch.arange(T)
    dh, Hh = c["head_dim"], c["heads"]
    f = 1.0 / 10000.0 ** (torch.arange(0, dh, 2).float() / dh)
    for i in range(c["layers"]):
        p = f"l{i}."
        h = plain.rms_norm(x, w[p + "n1"], c["eps"])
        if i % 2 == 0:
            u = h @ w[p + "state_w"].T
            s, ys = torch.zeros(c["width"]), []
            for t in range(T):
                s = c["decay"] * s + u[t]
                ys.append(s)
            x = x + torch.stack(ys)
            h = plain.rms_norm(x, w[p + "n2"], c["eps"])
            x = x + plain.swiglu(h, w[p + "gu"][: c["ffn"]].T, w[p + "gu"][c["ffn"]:].T, w[p + "down"].T)
        else:
            qkv = (h @ w[p + "qkv"].T).reshape(T, 3 * Hh, dh)
            q, k, v = qkv[:, :Hh], qkv[:, Hh:2 * Hh], qkv[:, 2 * Hh:]
            ang = pos.float()[:, None] * f[None]
            s_, c_ = torch.sin(ang)[:, None], torch.cos(ang)[:, None]
            rot = lambda z: torch.cat([z[..., : dh // 2] * c_ - z[..., dh // 2:] * s_, z[..., dh // 2:] * c_ + z[..., : dh // 2] * s_], -1)
            a = plain.gqa_attention(rot(q), rot(k), v, plain.attention_mask(pos, None, c["window"]))
            x = x + a.reshape(T, -1) @ w[p + "o"].T
            h = plain.rms_norm(x, w[p + "n2"], c["eps"])
            pr = torch.softmax(h @ w[p + "router"].T, -1)
            best = pr.argmax(-1)
            y = torch.zeros_like(h)
            for t in range(T):
                e = int(best[t])
                gu = w[p + f"e{e}.gu"]
                y[t] = plain.swiglu(h[t:t + 1], gu[: c["ffn"]].T, gu[c["ffn"]:].T, w[p + f"e{e}.down"].T)[0] * pr[t, e]
            x = x + y
    return plain.rms_norm(x, w["norm"], c["eps"]) @ w["head"].T


def test_a_toy_architecture_with_a_state_mixer_is_registered_built_and_stepped(tmp_path):
    J = _register_toy()
    from safetensors.torch import load_file

    folder = J.write_random_model(tmp_path / "toy", TOY, seed=5, dtype=torch.float32, std=0.15, norm_noise=0.1)
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyStateForCausalLM"]
    w = load_file(str(folder / "model.safetensors"))
    model = J.load_model(folder, "float32", DEV)
    assert len(model.plan.states) == 2 and len(model.plan.caches) == 2
    assert model.plan.groups[0].kind == J.cache.KEEP_WINDOW
    eng = J.Engine(model, max_tokens=3 * 64, page_size=8, max_slots=4)
    rng = random.Random(2)
    reqs = H.random_requests(rng, TOY["vocab_size"], [50, 9, 33, 41, 27])
    for steps in (H.trace_whole(reqs), H.trace_portions(reqs, rng), H.trace_mixed(reqs, rng, max_live=3)):
        got, _ = H.run_trace(eng, steps)
        for rid, toks in reqs.items():
            ref = _toy_plain(w, TOY, toks).numpy()
            for pos in range(len(toks)):
                err = H.rel_err(got[(rid, pos)], ref[pos])
                assert err < 2e-5, (rid, pos, err)
    # the windowed cache group gave pages back while requests ran, and everything is free at the end
    assert all(eng.manager.free_pages(g) == eng.num_pages for g in range(len(eng.manager.groups)))
    J.config.unregister_architecture("ToyStateForCausalLM")


# --------------------------------------------------------------------- the order of layers is data
def _plain_scheduled(cfg, w, toks, schedule):
    """Plain forward of Llama-4 blocks run in `schedule` order; an entry (block, source) with source != None
    takes keys and values from the earlier entry `source` instead of computing its own."""
    T = len(toks)
    x = w["model.embed_tokens.weight"][torch.tensor(toks)]
    pos = torch.arange(T)
    f = plain.rope_inverse_frequencies(cfg)
    Hq, Hkv, dh, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    kept = {}
    for entry, (i, source) in enumerate(schedule):
        p = f"model.layers.{i}."
        h = plain.rms_norm(x, w[p + "input_layernorm.weight"], eps)
        q = (h @ w[p + "self_attn.q_proj.weight"].T).reshape(T, Hq, dh)
        k = (h @ w[p + "self_attn.k_proj.weight"].T).reshape(T, Hkv, dh)
        v = (h @ w[p + "self_attn.v_proj.weight"].T).reshape(T, Hkv, dh)
        rope = plain.layer_uses_rope(cfg, i)
        if rope:
            q, k = plain.apply_rope_interleaved(q, pos, f), plain.apply_rope_interleaved(k, pos, f)
            if cfg["use_qk_norm"]:
                q, k = plain.rms_norm(q, None, eps), plain.rms_norm(k, None, eps)
        else:
            q = q * plain.attention_temperature(pos, cfg["floor_scale"], cfg["attn_scale"])[:, None, None]
        if source is not None:
            k, v = kept[source]
        kept[entry] = (k, v)
        a = plain.gqa_attention(q, k, v, plain.attention_mask(pos, cfg["attention_chunk_size"] if rope else None))
        x = x + a.reshape(T, -1) @ w[p + "self_attn.o_proj.weight"].T
        h = plain.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        pf = p + "feed_forward."
        if plain.layer_is_moe(cfg, i):
            y, _ = plain.moe(h, w[pf + "router.weight"].T, w[pf + "experts.gate_up_proj"], w[pf + "experts.down_proj"],
                             w[pf + "shared_expert.gate_proj.weight"].T, w[pf + "shared_expert.up_proj.weight"].T,
                             w[pf + "shared_expert.down_proj.weight"].T, cfg["num_experts_per_tok"])
        else:
            y = plain.swiglu(h, w[pf + "gate_proj.weight"].T, w[pf + "up_proj.weight"].T, w[pf + "down_proj.weight"].T)
        x = x + y
    return plain.rms_norm(x, w["model.norm.weight"], eps) @ w["lm_head.weight"].T


def test_a_block_run_twice_and_a_layer_reading_another_layers_cache(model_dirs):
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.parts import DecoderModel, LayerRun

    folder = model_dirs["tiny_b"]
    base = J.load_model(folder, "float32", DEV)
    # block 1 runs twice (own cache each time); the run of block 4 reads the cache that block 0 filled
    # (both rotary layers: same retention); block 3 (NoPE) runs once.
    schedule = [LayerRun(0, 0, True), LayerRun(1, 1, True), LayerRun(3, 2, True), LayerRun(1, 3, True), LayerRun(4, 0, False)]
    model = DecoderModel(base.runtime, base.embedding, base.blocks, base.final_norm, base.lm_head, schedule, base.config)
    assert len(model.plan.caches) == 4
    eng = J.Engine(model, max_tokens=256, page_size=16, max_slots=4)
    cfg, w = plain.load_config(folder), plain.load_weights(folder)
    rng = random.Random(9)
    reqs = H.random_requests(rng, 384, [70, 20, 55])
    plain_sched = [(0, None), (1, None), (3, None), (1, None), (4, 0)]
    for steps in (H.trace_whole(reqs), H.trace_mixed(reqs, rng, max_live=3)):
        got, _ = H.run_trace(eng, steps)
        for rid, toks in reqs.items():
            ref = _plain_scheduled(cfg, w, toks, plain_sched).numpy()
            worst = max(H.rel_err(got[(rid, p)], ref[p]) for p in range(len(toks)))
            assert worst < 2e-5, (rid, worst)
    with pytest.raises(ValueError, match="before any entry fills it"):
        DecoderModel(base.runtime, base.embedding, base.blocks, base.final_norm, base.lm_head,
                     [LayerRun(0, 0, False)], base.config)
    with pytest.raises(ValueError, match="already has a writer"):
        DecoderModel(base.runtime, base.embedding, base.blocks, base.final_norm, base.lm_head,
                     [LayerRun(0, 0, True), LayerRun(1, 0, True)], base.config)


# ------------------------------------------------------- per-request state under replayed CUDA graphs
def test_a_state_mixer_decodes_through_replayed_graphs():
    """A recurrent mixer whose decode step indexes its state slab by the descriptor's slot ids (device data) is
    captured and replayed like any other model: the replayed steps give the same logits, bit for bit, as the
    uncaptured ones.  A mixer that reads the step's host copies while being captured is refused loudly, and one
    that says so (``capturable = False``) is simply never captured."""
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.parts import DecoderModel, DenseSwiGLU, Mixer, PreNormBlock, RMSNorm, Runtime, StateNeed

    class DecayState(Mixer):
        def __init__(self, w, decay, mode):
            self.w, self.decay, self.mode = w.float(), float(decay), mode
            self.capturable = mode != "opts_out"

        def state_need(self):
            return StateNeed((self.w.shape[0],), torch.float32)

        def forward(self, ctx, h, cache):
            u = h.float() @ self.w.T
            if ctx.max_q_len == 1 and self.mode == "device":  # a decode step: state rows by the device's slot ids
                slots = ctx.slot_ids.long()
                s = self.decay * cache.state.index_select(0, slots) + u
                cache.state.index_copy_(0, slots, s)
                return s
            out, at = torch.empty_like(u), 0
            for n, slot in zip(ctx.host_q_lens, ctx.host_slot_ids):  # portions: planned on the host (never captured)
                s = cache.state[slot]
                for i in range(n):
                    s = self.decay * s + u[at + i]
                    out[at + i] = s
                cache.state[slot] = s
                at += n
            return out

    D, F, V = 64, 128, 50
    g = torch.Generator().manual_seed(4)
    r = lambda *shape: (torch.randn(*shape, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    rt = Runtime(torch.bfloat16, torch.device(DEV))

    def model(mode):
        torch.manual_seed(0)
        blocks = [PreNormBlock(RMSNorm(torch.ones(D, device=DEV), 1e-5), DecayState(w, 0.7, mode), RMSNorm(torch.ones(D, device=DEV), 1e-5),
                               DenseSwiGLU(gu, dn)) for w, gu, dn in weights]
        return DecoderModel(rt, emb, blocks, RMSNorm(torch.ones(D, device=DEV), 1e-5), head)

    weights = [(r(D, D), r(2 * F, D), r(D, F)) for _ in range(2)]
    emb, head = r(V, D), r(V, D)

    def run(mode, use_graphs, steps=12):
        eng = J.Engine(model(mode), max_tokens=64, page_size=16, max_slots=4, use_graphs=use_graphs)
        slots = [eng.new_request() for _ in range(3)]
        rows = [eng.step([J.StepEntry(s, [1 + i, 2, 3 + i], [2]) for i, s in enumerate(slots)]).clone()]
        for t in range(steps):
            rows.append(eng.step([J.StepEntry(s, [(5 * t + i) % V], [0]) for i, s in enumerate(slots)]).clone())
        eng.check_status()
        return torch.stack(rows), eng

    plain_rows, _ = run("device", False)
    graph_rows, eng = run("device", True)
    assert eng.graph_replays >= 10
    assert torch.equal(plain_rows, graph_rows)
    with pytest.raises(J.EngineError, match="capturable"):
        run("host", True)
    rows, eng = run("opts_out", True)
    assert eng.graph_replays == 0 and torch.equal(rows, plain_rows)
