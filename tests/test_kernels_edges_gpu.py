"""Edges and long positions of the kernels, where random inputs would hide a fault: the first position a query
may see (chunk starts and window edges) inside and across the tcgen05 kernel's 128-row query tiles, portions that
start anywhere after cached history, tiles whose last rows belong to another request, block-table holes left by
released pages, rotation angles at positions up to 131071, and every attention kernel at a context of 32768
tokens with the real chunk (8192) and temperature floor (8192)."""

import pytest
import torch

from tests.test_kernels_gpu import DEV, K, _attention_ref, close, status

pytestmark = pytest.mark.gpu


def _case(dtype, Hq, Hkv, dh, page, lens, q_lens, seed=0, q_gain=1.0, holes_before=None):
    """Requests with `lens` tokens in a paged cache (random page order), the last `q_lens` of each being this step's
    queries.  Returns q, pages, block table, req_of_token, positions and each request's keys and values [L, Hkv, dh].
    ``holes_before``: per request, block-table entries of pages wholly before that position are -1 (released)."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    R = len(lens)
    width = max(-(-L // page) for L in lens)
    P = R * width + 3
    ids = torch.randperm(P, generator=torch.Generator().manual_seed(seed))[: R * width].to(torch.int32).reshape(R, width).to(DEV)
    pages = torch.randn(P, 2, Hkv, page, dh, device=DEV, generator=g).to(dtype)
    ks, vs = [], []
    for r, L in enumerate(lens):
        p = torch.arange(L, device=DEV)
        pg, slot = ids[r, p // page].long(), p % page
        ks.append(pages[pg, 0, :, slot]), vs.append(pages[pg, 1, :, slot])
    pos = torch.cat([torch.arange(L - n, L, device=DEV, dtype=torch.int32) for L, n in zip(lens, q_lens)])
    req = torch.cat([torch.full((n,), r, device=DEV, dtype=torch.int32) for r, n in enumerate(q_lens)])
    q = (torch.randn(len(pos), Hq, dh, device=DEV, generator=g) * q_gain).to(dtype)
    if holes_before is not None:
        for r, first in enumerate(holes_before):
            ids[r, : first // page] = -1
    return q, pages, ids, req, pos, ks, vs


def _tiles(q_lens, rows):
    t, at = [], 0
    for n in q_lens:
        t += [(at + o, min(rows, n - o)) for o in range(0, n, rows)]
        at += n
    return torch.tensor(t, device=DEV, dtype=torch.int32)


def _first_visible(p, chunk, window):
    lo = 0
    if chunk:
        lo = p - p % chunk
    if window:
        lo = max(lo, p - window + 1)
    return lo


def _run_tc(q, pages, bt, req, pos, q_lens, chunk, window, temp=(0.0, 1.0)):
    out, st = torch.full_like(q, float("nan")), status()
    tl = _tiles(q_lens, 128)
    K().attention_prefill_tc(q, pages, bt, req, pos, out, tl, len(tl), q.shape[-1] ** -0.5, chunk, window, temp[0], temp[1], st)
    torch.cuda.synchronize()
    assert int(st) == 0
    return out


# (page, chunk, window, cached tokens before the portion, tokens of the portion)
TC_EDGE_CASES = [
    (64, 192, 0, 2 * 128 + 37, 300),   # portion starts at k * 128 + 37; tiles straddle chunk starts at 384 and 576
    (128, 192, 0, 37, 420),            # pages of 128 keys
    (64, 0, 100, 128 + 37, 260),       # a window: every row has its own first visible key
    (64, 128, 0, 0, 384),              # chunk = tile height, aligned: whole tiles before the chunk start are skipped
    (128, 320, 150, 200, 300),         # chunk and window at once
]


@pytest.mark.parametrize("page, chunk, window, before, n", TC_EDGE_CASES)
def test_tcgen05_attention_sees_exactly_the_keys_it_may(page, chunk, window, before, n):
    """One key whose score swamps all others, placed in turn on every edge: the first position some row may see,
    the one before it, page and tile boundaries.  A row that may see it returns that key's value (1000), a row that
    may not must not contain it at all; and every row agrees with the 32-bit reference."""
    Hq, Hkv, dh = 4, 2, 128
    L = before + n
    edges = {0, 63, 64, 127, 128, before - 1, before, before + 127, before + 128, L - 1}
    for p in (before, before + 127, before + 128, L - 1):
        lo = _first_visible(p, chunk, window)
        edges |= {lo, lo - 1}
    if chunk:
        edges |= {c for c in range(chunk, L, chunk)} | {c - 1 for c in range(chunk, L, chunk)}
    for hot in sorted(e for e in edges if 0 <= e < L):
        q, pages, bt, req, pos, ks, vs = _case(torch.bfloat16, Hq, Hkv, dh, page, [L], [n], seed=hot)
        pg, slot = int(bt[0, hot // page]), hot % page
        pages[pg, 0, :, slot] = 0
        pages[pg, 0, :, slot, 0] = 40.0
        pages[pg, 1, :, slot] = 1000.0
        ks[0][hot], vs[0][hot] = pages[pg, 0, :, slot], pages[pg, 1, :, slot]
        q[:] = 0
        q[..., 0] = 40.0  # score 1600 / sqrt(128) = 141 for the hot key, 0 for the others
        out = _run_tc(q, pages, bt, req, pos, [n], chunk, window).float()
        for i, p in enumerate(pos.tolist()):
            sees = _first_visible(p, chunk, window) <= hot <= p
            if sees:
                assert float((out[i] - 1000.0).abs().max()) < 10.0, f"hot key {hot}: the row at position {p} should see it"
            else:
                assert float(out[i].abs().max()) < 10.0, f"hot key {hot}: the row at position {p} must not see it"
        ref = _attention_ref(q, ks[0], vs[0], pos.long(), chunk, window, dh ** -0.5, 0.0, 1.0)
        close(out, ref, 1.5e-2)


def test_tcgen05_attention_tiles_that_end_inside_another_requests_rows():
    """Tiles of fewer than 128 rows: the query load brings the next request's rows into the tile, which must be
    neither used nor written; the last request's last tile reaches beyond the end of q."""
    Hq, Hkv, dh, page = 10, 2, 128, 64
    lens, q_lens = [400, 100, 250, 64], [100, 100, 150, 64]
    q, pages, bt, req, pos, ks, vs = _case(torch.bfloat16, Hq, Hkv, dh, page, lens, q_lens, seed=3, q_gain=3.0)
    out = _run_tc(q, pages, bt, req, pos, q_lens, 256, 0, (0.1, 64.0))
    at = 0
    for r, n in enumerate(q_lens):
        ref = _attention_ref(q[at:at + n], ks[r], vs[r], pos[at:at + n].long(), 256, 0, dh ** -0.5, 0.1, 64.0)
        close(out[at:at + n], ref, 1.5e-2)
        at += n
    # only some of the requests listed: the rows of the others stay untouched
    out2 = torch.full_like(q, 7.0)
    st = status()
    tl = _tiles(q_lens, 128)
    keep = tl[(tl[:, 0] >= 200) & (tl[:, 0] < 350)].contiguous()  # the third request's two tiles
    K().attention_prefill_tc(q, pages, bt, req, pos, out2, keep, len(keep), dh ** -0.5, 256, 0, 0.1, 64.0, st)
    assert int(st) == 0
    assert torch.equal(out2[200:350], out[200:350])
    assert bool((out2[:200] == 7.0).all()) and bool((out2[350:] == 7.0).all())


@pytest.mark.parametrize("page", [64, 128])
def test_attention_kernels_with_released_pages_before_the_chunk(page):
    """After a request crossed a chunk start the cache manager gives the old chunk's pages back: the block table
    holds -1 there.  No kernel may read through such an entry; page 0, which a careless kernel would read
    instead, holds a key that would swamp everything."""
    # The chunk start (576) is no multiple of the key tile (128): with pages of 64 the released page 512..575 lies
    # inside the first key tile that the tcgen05 kernel fetches.
    Hq, Hkv, dh, chunk = 4, 2, 128, 576
    L, n = chunk + 300, 200  # the portion's rows lie at 676..875, all in the second chunk
    api = K()
    q, pages, bt, req, pos, ks, vs = _case(torch.bfloat16, Hq, Hkv, dh, page, [L], [n], seed=5, holes_before=[chunk])
    if 0 in bt[0].tolist():  # page 0 must be nobody's: move its tokens to a page that the table does not name
        spare = next(i for i in range(pages.shape[0]) if i not in bt[0].tolist())
        pages[spare] = pages[0]
        bt[0, bt[0].tolist().index(0)] = spare
    assert int(bt[0, 0]) == -1 and 0 not in bt[0].tolist()
    pages[0, 0] = 0
    pages[0, 0, :, :, 0] = 40.0
    pages[0, 1] = 1000.0
    q[..., 0] = 40.0
    ref = _attention_ref(q, ks[0], vs[0], pos.long(), chunk, 0, dh ** -0.5, 0.0, 1.0)
    close(_run_tc(q, pages, bt, req, pos, [n], chunk, 0), ref, 1.5e-2)
    out, st = torch.full_like(q, float("nan")), status()
    tl = _tiles([n], 16)
    api.attention_prefill(q, pages, bt, req, pos, out, tl, len(tl), dh ** -0.5, chunk, 0, 0.0, 1.0, st)
    close(out, ref, 1.5e-2)
    out.fill_(float("nan"))
    api.attention_generic(q, pages, bt, req, pos, out, dh ** -0.5, chunk, 0, 0.0, 1.0, st)
    close(out, ref, 1.5e-2)
    # the last row alone, as a decoded token
    keys, splits = api.attention_decode_plan(L, chunk, 0, Hkv)
    part_o, part_ml = torch.empty(Hq * splits * dh, device=DEV), torch.empty(Hq * splits * 2, device=DEV)
    o1 = torch.empty_like(q[-1:])
    api.attention_decode(q[-1:].contiguous(), pages, bt, req[-1:].contiguous(), pos[-1:].contiguous(), o1, dh ** -0.5, chunk, 0,
                         0.0, 1.0, part_o, part_ml, splits, keys, st)
    close(o1, ref[-1:], 1.5e-2)
    assert int(st) == 0


# ------------------------------------------------------------------------------- long positions
def _rope64(x, ang):
    s, c = torch.sin(ang)[:, None], torch.cos(ang)[:, None]
    a, b = x[..., 0::2].double(), x[..., 1::2].double()
    return torch.stack([a * c - b * s, b * c + a * s], -1).reshape(x.shape)


@pytest.mark.parametrize("n_tokens", [4, 80])  # one head per warp (a decode step's few rows), several (a portion)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_at_long_positions(dtype, n_tokens):
    """Positions 32767, 32768, 65535 and 131071 (and portions that end there).  The angle p * f is a 32-bit
    product, as in the reference (model.py:706-709): near 131071 radians its spacing is 2^-7, so against angles
    computed in 64-bit a rotated element may differ by 2^-8 of the pair's length; against the same 32-bit angle
    with sine and cosine taken in 64-bit, only by the rounding of a 32-bit sine."""
    Hq, Hkv, dh, page = 8, 2, 128, 64
    from jax_llm_examples_b200.parts import llama3_scaled_frequencies

    inv_freq = llama3_scaled_frequencies(dh, 500000.0, {"factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                                                        "original_max_position_embeddings": 8192}).to(DEV)
    for last in (32767, 32768, 65535, 131071):
        pos = torch.arange(last - n_tokens + 1, last + 1, device=DEV, dtype=torch.int32)
        req = torch.zeros(n_tokens, device=DEV, dtype=torch.int32)
        width = last // page + 1
        bt = torch.full((1, width), -1, device=DEV, dtype=torch.int32)
        first_page = int(pos[0]) // page
        n_pages = width - first_page
        bt[0, first_page:] = torch.randperm(n_pages + 2)[:n_pages].to(torch.int32).to(DEV)
        pages = torch.zeros(n_pages + 2, 2, Hkv, page, dh, device=DEV, dtype=dtype)
        qkv = torch.randn(n_tokens, (Hq + 2 * Hkv) * dh, device=DEV).to(dtype)
        q_out, st = torch.empty(n_tokens, Hq, dh, device=DEV, dtype=dtype), status()
        K().rope_kv_store(qkv, q_out, pages, bt, req, pos, inv_freq, False, 1.0, Hq, Hkv, dh, st)
        assert int(st) == 0
        x = qkv.float().reshape(n_tokens, Hq + 2 * Hkv, dh)
        ang32 = (pos.float()[:, None] * inv_freq[None]).double()       # the 32-bit product, then exact
        ang64 = pos.double()[:, None] * inv_freq.double()[None]        # everything exact
        k_got = pages[bt[0, (pos // page).long()].long(), 0, :, (pos % page).long()]
        for got, src in ((q_out, x[:, :Hq]), (k_got, x[:, Hq:Hq + Hkv])):
            tight, loose = (3e-6, 2.0 ** -8 * 1.5) if dtype == torch.float32 else (8e-3, 1.2e-2)
            close(got, _rope64(src, ang32), tight)
            close(got, _rope64(src, ang64), loose)


def _long_context_case(dtype, Hq, Hkv, n_q, last, page=64, seed=0):
    """One request holding positions 0..last in the cache; its last n_q tokens are the step's queries."""
    return _case(dtype, Hq, Hkv, 128, page, [last + 1], [n_q], seed=seed, q_gain=4.0)


LONG = 32768
# a rotary layer (chunk 8192, no temperature) and a NoPE layer (all keys, temperature with floor 8192: the factor
# floor((p + 1) / 8192) reaches 4 at the last position)
LAYER_KINDS = [("chunked", 8192, 0.0, 1.0), ("global_with_temperature", 0, 0.1, 8192.0)]


@pytest.mark.parametrize("kind, chunk, attn_scale, floor_scale", LAYER_KINDS)
def test_decode_attention_at_32768_tokens(kind, chunk, attn_scale, floor_scale):
    Hq, Hkv, dh = 10, 2, 128
    api = K()
    for last in (LONG - 1, 3 * 8192, 3 * 8192 - 1):  # the end; the first position of a chunk; the last of one
        q, pages, bt, req, pos, ks, vs = _long_context_case(torch.bfloat16, Hq, Hkv, 1, last, seed=last)
        ref = _attention_ref(q, ks[0], vs[0], pos.long(), chunk, 0, dh ** -0.5, attn_scale, floor_scale)
        for pairs in (Hkv, 64 * Hkv):  # many short splits; few long ones
            keys, splits = api.attention_decode_plan(last + 1, chunk, 0, pairs)
            part_o, part_ml = torch.empty(Hq * splits * dh, device=DEV), torch.empty(Hq * splits * 2, device=DEV)
            out, st = torch.full_like(q, float("nan")), status()
            api.attention_decode(q, pages, bt, req, pos, out, dh ** -0.5, chunk, 0, attn_scale, floor_scale, part_o, part_ml,
                                 splits, keys, st)
            assert int(st) == 0
            close(out, ref, 1.5e-2)
        out, st = torch.full_like(q, float("nan")), status()
        api.attention_generic(q, pages, bt, req, pos, out, dh ** -0.5, chunk, 0, attn_scale, floor_scale, st)
        close(out, ref, 1.5e-2)


@pytest.mark.parametrize("kind, chunk, attn_scale, floor_scale", LAYER_KINDS)
def test_prompt_attention_at_32768_tokens(kind, chunk, attn_scale, floor_scale):
    """A portion of 300 tokens that ends at position 32767, and one that crosses the chunk start at 24576; the
    tcgen05 kernel, the mma.sync flash kernel and the generic kernel (bfloat16 and 32-bit)."""
    Hq, Hkv, dh = 10, 2, 128
    api = K()
    for last in (LONG - 1, 3 * 8192 + 130):
        n = 300
        q, pages, bt, req, pos, ks, vs = _long_context_case(torch.bfloat16, Hq, Hkv, n, last, seed=last)
        ref = _attention_ref(q, ks[0], vs[0], pos.long(), chunk, 0, dh ** -0.5, attn_scale, floor_scale)
        close(_run_tc(q, pages, bt, req, pos, [n], chunk, 0, (attn_scale, floor_scale)), ref, 1.5e-2)
        out, st = torch.full_like(q, float("nan")), status()
        tl = _tiles([n], 16)
        api.attention_prefill(q, pages, bt, req, pos, out, tl, len(tl), dh ** -0.5, chunk, 0, attn_scale, floor_scale, st)
        close(out, ref, 1.5e-2)
        out.fill_(float("nan"))
        api.attention_generic(q, pages, bt, req, pos, out, dh ** -0.5, chunk, 0, attn_scale, floor_scale, st)
        close(out, ref, 1.5e-2)
        assert int(st) == 0
    # 32-bit: the generic kernel on a short portion at the far end
    q, pages, bt, req, pos, ks, vs = _long_context_case(torch.float32, 4, 2, 40, LONG - 1, seed=9)
    ref = _attention_ref(q, ks[0], vs[0], pos.long(), chunk, 0, dh ** -0.5, attn_scale, floor_scale)
    out, st = torch.full_like(q, float("nan")), status()
    api.attention_generic(q, pages, bt, req, pos, out, dh ** -0.5, chunk, 0, attn_scale, floor_scale, st)
    assert int(st) == 0
    close(out, ref, 1e-5)
