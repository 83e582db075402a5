"""Each CUDA kernel alone against a plain float32 torch reference of the same operation, at sizes
other than the engine's: odd widths, head sizes in steps of 16, any head and group counts."""

import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def K():
    from jax_llm_examples_b200.kernels import api

    return api


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def close(a, b, tol):
    err = float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))
    assert err < tol, f"relative error {err:.3e} (tolerance {tol})"
    return err


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V, D, N", [(1000, 72, 5), (257, 1030, 33)])
def test_embed(dtype, V, D, N):
    table = torch.randn(V, D, device=DEV).to(dtype)
    ids = torch.randint(0, V, (N,), device=DEV, dtype=torch.int32)
    x, st = torch.empty(N, D, device=DEV), status()
    K().embed(ids, table, x, st)
    assert torch.equal(x, table[ids.long()].float()) and int(st) == 0
    ids[0] = V  # outside the vocabulary: flagged, not read
    K().embed(ids, table, x, st)
    assert int(st) == 2


@pytest.mark.parametrize("out_dtype, tol", [(torch.float32, 2e-6), (torch.bfloat16, 5e-3)])
@pytest.mark.parametrize("N, D, eps", [(7, 96, 1e-6), (3, 5120, 1e-5), (130, 1000, 1e-3)])
def test_add_rmsnorm(out_dtype, tol, N, D, eps):
    x, delta, g = torch.randn(N, D, device=DEV), torch.randn(N, D, device=DEV), 1 + 0.1 * torch.randn(D, device=DEV)
    s = x + delta
    ref = g * s / torch.sqrt((s * s).mean(-1, keepdim=True) + eps)
    xc, out, out32 = x.clone(), torch.empty(N, D, device=DEV, dtype=out_dtype), torch.empty(N, D, device=DEV)
    K().add_rmsnorm(xc, delta, g, eps, out, out32)
    close(out, ref, tol), close(out32, ref, 2e-6)
    assert torch.equal(xc, s)  # the residual sum is written back
    # weightless, no delta, gathered rows
    rows = torch.tensor([N - 1, 0, N // 2], device=DEV, dtype=torch.int32)
    out2 = torch.empty(3, D, device=DEV, dtype=out_dtype)
    xc2 = x.clone()
    K().add_rmsnorm(xc2, delta, None, eps, out2, None, rows)
    sr = s[rows.long()]
    close(out2, sr / torch.sqrt((sr * sr).mean(-1, keepdim=True) + eps), tol)
    assert torch.equal(xc2, x)  # gathered rows are not written back


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 1e-6), (torch.bfloat16, 1e-2)])
def test_silu_mul(dtype, tol):
    gu = torch.randn(9, 2 * 200, device=DEV).to(dtype)
    out = torch.empty(9, 200, device=DEV, dtype=dtype)
    K().silu_mul(gu, out)
    g, u = gu.float()[:, :200], gu.float()[:, 200:]
    close(out, torch.nn.functional.silu(g) * u, tol)


def _rope_ref(x, pos, inv_freq):
    ang = pos.float()[:, None] * inv_freq[None]
    s, c = torch.sin(ang)[:, None], torch.cos(ang)[:, None]
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * c - b * s, b * c + a * s], -1).reshape(x.shape)


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 3e-6), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("Hq, Hkv, dh, page, rope, l2", [(6, 3, 48, 8, True, True), (5, 1, 16, 4, True, False),
                                                         (4, 4, 112, 16, False, False), (8, 2, 256, 32, True, True)])
def test_rope_kv_store(dtype, tol, Hq, Hkv, dh, page, rope, l2):
    N, P, eps = 11, 9, 1e-5
    qkv = torch.randn(N, (Hq + 2 * Hkv) * dh, device=DEV).to(dtype)
    # two requests: tokens 0..5 at positions 20..25 of request 0; tokens 6..10 at positions 0..4 of request 1
    pos = torch.tensor(list(range(20, 26)) + list(range(5)), device=DEV, dtype=torch.int32)
    req = torch.tensor([0] * 6 + [1] * 5, device=DEV, dtype=torch.int32)
    width = 26 // page + 1
    perm = torch.randperm(P)[: 2 * width].to(torch.int32).reshape(2, width) if 2 * width <= P else None
    if perm is None:
        P = 2 * width
        perm = torch.randperm(P).to(torch.int32).reshape(2, width)
    bt = perm.to(DEV)
    pages = torch.zeros(P, 2, Hkv, page, dh, device=DEV, dtype=dtype)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, dh, 2, device=DEV).float() / dh))) if rope else None
    q_out, st = torch.empty(N, Hq, dh, device=DEV, dtype=dtype), status()
    K().rope_kv_store(qkv, q_out, pages, bt, req, pos, inv_freq, l2, eps, Hq, Hkv, dh, st)
    assert int(st) == 0
    x = qkv.float().reshape(N, Hq + 2 * Hkv, dh)
    q, k, v = x[:, :Hq], x[:, Hq:Hq + Hkv], x[:, Hq + Hkv:]
    if rope:
        q, k = _rope_ref(q, pos, inv_freq), _rope_ref(k, pos, inv_freq)
    if l2:
        q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps)
        k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps)
    close(q_out, q, tol)
    for n in range(N):
        pg = int(bt[int(req[n]), int(pos[n]) // page])
        slot = int(pos[n]) % page
        close(pages[pg, 0, :, slot], k[n], tol)
        assert torch.equal(pages[pg, 1, :, slot].float(), v[n])
    # a block-table entry outside the pool is flagged and nothing is written there
    bt2 = bt.clone()
    bt2[0, 20 // page] = P + 3
    K().rope_kv_store(qkv, q_out, pages, bt2, req, pos, inv_freq, l2, eps, Hq, Hkv, dh, st)
    assert int(st) == 1


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 3e-6), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("Hq, Hkv, dh, page, l2", [(40, 8, 128, 64, True), (9, 3, 48, 16, False), (3, 1, 320, 32, True),
                                                   (10, 2, 64, 16, True), (5, 5, 16, 8, False), (4, 1, 256, 64, True)])
def test_rope_kv_store_many_tokens(dtype, tol, Hq, Hkv, dh, page, l2):
    """A prompt portion: 300 tokens of one request from position 70 on (several heads per warp; in bfloat16 with a
    head size of 8 times a power of two, the kernel that takes a token's heads 16 bytes at a time)."""
    N, eps, first = 300, 1e-5, 70
    qkv = torch.randn(N, (Hq + 2 * Hkv) * dh, device=DEV).to(dtype)
    pos = torch.arange(first, first + N, device=DEV, dtype=torch.int32)
    req = torch.zeros(N, device=DEV, dtype=torch.int32)
    width = (first + N - 1) // page + 1
    bt = torch.randperm(width + 3)[:width].to(torch.int32).reshape(1, width).to(DEV)
    pages = torch.zeros(width + 3, 2, Hkv, page, dh, device=DEV, dtype=dtype)
    inv_freq = 1.0 / (500000.0 ** (torch.arange(0, dh, 2, device=DEV).float() / dh))
    q_out, st = torch.full((N, Hq, dh), float("nan"), device=DEV, dtype=dtype), status()
    K().rope_kv_store(qkv, q_out, pages, bt, req, pos, inv_freq, l2, eps, Hq, Hkv, dh, st)
    assert int(st) == 0
    x = qkv.float().reshape(N, Hq + 2 * Hkv, dh)
    q, k, v = _rope_ref(x[:, :Hq], pos, inv_freq), _rope_ref(x[:, Hq:Hq + Hkv], pos, inv_freq), x[:, Hq + Hkv:]
    if l2:
        q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps)
        k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps)
    close(q_out, q, tol)
    pg, slot = bt[0, (pos // page).long()].long(), (pos % page).long()
    close(pages[pg, 0, :, slot], k, tol)
    assert torch.equal(pages[pg, 1, :, slot].float(), v)


def _attention_ref(q, k_all, v_all, q_pos, chunk, window, scale, attn_scale, floor_scale):
    """q: [n, Hq, dh] at positions q_pos of one request; k_all, v_all: [S, Hkv, dh] for positions 0..S-1."""
    n, Hq, dh = q.shape
    Hkv = k_all.shape[1]
    G = Hq // Hkv
    S = k_all.shape[0]
    kp = torch.arange(S, device=q.device)
    mask = q_pos[:, None] >= kp[None]
    if chunk:
        mask &= (q_pos[:, None] // chunk) == (kp[None] // chunk)
    if window:
        mask &= (q_pos[:, None] - kp[None]) < window
    qs = q.float()
    if attn_scale:
        qs = qs * (1 + attn_scale * torch.log1p(torch.floor((q_pos.float() + 1) / floor_scale)))[:, None, None]
    s = torch.einsum("nhgd,shd->hgns", qs.reshape(n, Hkv, G, dh), k_all.float()) * scale
    s = s.masked_fill(~mask[None, None], float("-inf"))
    return torch.einsum("hgns,shd->nhgd", torch.softmax(s, -1), v_all.float()).reshape(n, Hq, dh)


def _paged_case(dtype, Hq, Hkv, dh, page, lens, q_lens, seed=0):
    """Requests with `lens` tokens in the cache, the last `q_lens` of them being this step's queries."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    R = len(lens)
    width = max(-(-L // page) for L in lens)
    P = R * width + 3
    ids = torch.randperm(P, generator=torch.Generator().manual_seed(seed))[: R * width].to(torch.int32).reshape(R, width)
    pages = torch.randn(P, 2, Hkv, page, dh, device=DEV, generator=g).to(dtype)
    ks, vs = [], []
    for r, L in enumerate(lens):
        k = torch.stack([pages[int(ids[r, p // page]), 0, :, p % page] for p in range(L)])
        v = torch.stack([pages[int(ids[r, p // page]), 1, :, p % page] for p in range(L)])
        ks.append(k), vs.append(v)
    pos = torch.tensor([p for L, n in zip(lens, q_lens) for p in range(L - n, L)], device=DEV, dtype=torch.int32)
    req = torch.tensor([r for r, n in enumerate(q_lens) for _ in range(n)], device=DEV, dtype=torch.int32)
    q = torch.randn(len(pos), Hq, dh, device=DEV, generator=g).to(dtype)
    return q, pages, ids.to(DEV), req, pos, ks, vs


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 5e-6), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("Hq, Hkv, dh, page, chunk, window, temp", [
    (6, 2, 48, 8, 0, 0, False), (5, 5, 16, 4, 24, 0, False), (12, 1, 80, 16, 0, 13, True), (8, 2, 128, 64, 64, 0, True),
    (3, 3, 272, 16, 0, 0, False)])
def test_attention_generic(dtype, tol, Hq, Hkv, dh, page, chunk, window, temp):
    lens, q_lens = [150, 37, 1, 66], [40, 1, 1, 66]
    q, pages, bt, req, pos, ks, vs = _paged_case(dtype, Hq, Hkv, dh, page, lens, q_lens)
    out, st = torch.empty_like(q), status()
    attn_scale, floor_scale = (0.1, 16.0) if temp else (0.0, 1.0)
    K().attention_generic(q, pages, bt, req, pos, out, dh ** -0.5, chunk, window, attn_scale, floor_scale, st)
    assert int(st) == 0
    at = 0
    for r, n in enumerate(q_lens):
        ref = _attention_ref(q[at:at + n], ks[r], vs[r], pos[at:at + n].long(), chunk, window, dh ** -0.5, attn_scale, floor_scale)
        close(out[at:at + n], ref, tol)
        at += n


def test_attention_finds_one_far_key_among_hundreds():
    """Random keys would hide a key that is skipped or read from the wrong page: here one key far back
    matches the query strongly, so almost all of the output is that key's value."""
    Hq, Hkv, dh, page = 4, 2, 64, 16
    for dtype in (torch.float32, torch.bfloat16):
        for far in (0, 15, 16, 17, 255, 256, 511):
            q, pages, bt, req, pos, ks, vs = _paged_case(dtype, Hq, Hkv, dh, page, [600], [1], seed=far)
            pg, slot = int(bt[0, far // page]), far % page
            pages[pg, 0, :, slot] = 0
            pages[pg, 0, :, slot, 0] = 40.0
            q[:] = 0
            q[..., 0] = 40.0  # score 1600 / 8 = 200 for that key, ~0 for the others
            out, st = torch.empty_like(q), status()
            K().attention_generic(q, pages, bt, req, pos, out, dh ** -0.5, 0, 0, 0.0, 1.0, st)
            want = pages[pg, 1, :, slot].float().repeat_interleave(Hq // Hkv, 0)
            close(out[0], want, 1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("ta, tw, tc", [(torch.float32,) * 3, (torch.bfloat16, torch.float32, torch.float32),
                                        (torch.bfloat16, torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M, N, Kd", [(1, 130, 70), (65, 64, 16), (200, 333, 257)])
def test_gemm_simt(ta, tw, tc, M, N, Kd):
    a, w = torch.randn(M, Kd, device=DEV).to(ta), torch.randn(N, Kd, device=DEV).to(tw)
    out = torch.empty(M, N, device=DEV, dtype=tc)
    K().gemm_simt(a, w, out)
    close(out, a.double() @ w.double().T, 1e-2 if tc == torch.bfloat16 else 2e-6)


def _groups(E, sizes_seed, total):
    rng = random.Random(sizes_seed)
    cuts = sorted(rng.randrange(total + 1) for _ in range(E - 1))
    return torch.tensor([0] + cuts + [total], dtype=torch.int32)


@pytest.mark.parametrize("E, rows, N, Kd", [(4, 37, 70, 50), (8, 300, 130, 64), (3, 5, 64, 129)])
def test_gemm_simt_grouped(E, rows, N, Kd):
    a, w = torch.randn(rows, Kd, device=DEV), torch.randn(E, N, Kd, device=DEV)
    off = _groups(E, rows, rows)
    out = torch.full((rows, N), float("nan"), device=DEV)
    K().gemm_simt(a, w, out, off.to(DEV))
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            close(out[lo:hi], a[lo:hi].double() @ w[e].double().T, 2e-6)


@pytest.mark.parametrize("M, N, Kd, out_dtype, splits", [
    (1, 128, 64, torch.float32, 1), (8, 384, 512, torch.bfloat16, 1), (5, 200, 136, torch.float32, 1),
    (64, 1000, 1024, torch.float32, 1), (130, 256, 320, torch.bfloat16, 1), (300, 130, 72, torch.float32, 1),
    (8, 640, 2048, torch.float32, 4), (33, 130, 1000, torch.bfloat16, 3),
    # 96 rows and more with outputs in multiples of 256: pairs of blocks sharing each MMA (cta_group::2)
    (100, 256, 320, torch.float32, 1), (150, 512, 1096, torch.bfloat16, 1), (256, 768, 2048, torch.float32, 2),
    (203, 256, 64, torch.float32, 1)])
def test_gemm_stream_dense(M, N, Kd, out_dtype, splits):
    """The tcgen05 product against float64 of the same bfloat16 operands."""
    a = torch.randn(M, Kd, device=DEV).bfloat16()
    w = torch.randn(N, Kd, device=DEV).bfloat16()
    out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
    scratch = torch.empty(splits * M * N, device=DEV) if splits > 1 else None
    st = status()
    K().gemm_stream(a, w, out, st, splits=splits, scratch=scratch)
    torch.cuda.synchronize()
    assert int(st) == 0
    close(out, a.double() @ w.double().T, 1e-2 if out_dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("E, rows, N, Kd, hint", [(4, 37, 256, 128, 0), (16, 64, 384, 512, 4), (8, 700, 130, 200, 88),
                                                  (5, 9, 128, 64, 16), (6, 900, 512, 328, 150), (3, 500, 256, 1024, 250),
                                                  (7, 640, 768, 192, 100)])
def test_gemm_stream_grouped(E, rows, N, Kd, hint):
    a = torch.randn(rows, Kd, device=DEV).bfloat16()
    w = torch.randn(E, N, Kd, device=DEV).bfloat16()
    off = _groups(E, rows + 1, rows)
    out = torch.full((rows, N), float("nan"), device=DEV)
    st = status()
    K().gemm_stream(a, w, out, st, offsets=off.to(DEV), rows_hint=hint)
    torch.cuda.synchronize()
    assert int(st) == 0
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            close(out[lo:hi], a[lo:hi].double() @ w[e].double().T, 1e-5)


def test_gemm_stream_refuses_what_it_cannot_take():
    a, w = torch.randn(4, 70, device=DEV).bfloat16(), torch.randn(128, 70, device=DEV).bfloat16()
    with pytest.raises(K().KernelError, match="multiple of 8"):
        K().gemm_stream(a, w, torch.empty(4, 128, device=DEV), status())


@pytest.mark.parametrize("N, D, E, k", [(33, 96, 8, 2), (5, 5120, 16, 1), (64, 200, 128, 4), (1, 64, 3, 3)])
def test_router_and_sort(N, D, E, k):
    h, w = torch.randn(N, D, device=DEV), torch.randn(E, D, device=DEV)
    idx = torch.empty(N, k, device=DEV, dtype=torch.int32)
    wt, scores = torch.empty(N, k, device=DEV), torch.empty(N, E, device=DEV)
    K().router(h, w, idx, wt, scores)
    ref = h.double() @ w.double().T
    close(scores, ref, 5e-6)
    order = torch.sort(scores, dim=-1, descending=True, stable=True)
    assert torch.equal(idx.long(), order.indices[:, :k])
    close(wt, torch.sigmoid(order.values[:, :k]), 1e-6)
    off = torch.empty(E + 1, device=DEV, dtype=torch.int32)
    pair, pos, st = torch.empty(N * k, device=DEV, dtype=torch.int32), torch.empty(N * k, device=DEV, dtype=torch.int32), status()
    K().expert_sort(idx, off, pair, pos, E, st)
    flat = idx.flatten().long()
    counts = torch.bincount(flat, minlength=E)
    assert torch.equal(off.long(), torch.cat([torch.zeros(1, device=DEV, dtype=torch.long), counts.cumsum(0)]))
    assert torch.equal(pair.long(), torch.sort(flat, stable=True).indices)
    assert torch.equal(pos.long()[pair.long()], torch.arange(N * k, device=DEV)) and int(st) == 0


@pytest.mark.parametrize("N, E, k, extra, tile_rows", [(353, 40, 2, 0, 32), (64, 16, 1, 0, 16), (7, 40, 2, 7, 16), (200, 130, 3, 0, 16),
                                                       (300, 32, 1, 300, 64), (1, 31, 1, 1, 16)])
def test_expert_sort_lists_the_row_tiles_and_nothing_else(N, E, k, extra, tile_rows):
    """offsets, the stable order, and the list of row tiles (group, first row) of every group that has rows, with the
    appended group of a shared expert last; the entries of the list past the last tile stay untouched."""
    idx = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(N)]).to(torch.int32)
    P, groups = N * k, E + (extra > 0)
    off = torch.full((E + 2,), -7, device=DEV, dtype=torch.int32)
    pair, pos, st = torch.full((P,), -7, device=DEV, dtype=torch.int32), torch.full((P,), -7, device=DEV, dtype=torch.int32), status()
    tl = torch.full((2 * (-(-(P + extra) // tile_rows) + groups),), -7, device=DEV, dtype=torch.int32)
    nt = torch.full((1,), -7, device=DEV, dtype=torch.int32)
    K().expert_sort(idx, off, pair, pos, E, st, extra, tile_rows, tl, nt)
    flat = idx.flatten().long()
    bounds = [0] + torch.bincount(flat, minlength=E).cumsum(0).tolist() + ([P + extra] if extra else [])
    assert off[:len(bounds)].tolist() == bounds and int(st) == 0
    assert torch.equal(pair.long(), torch.sort(flat, stable=True).indices)
    assert torch.equal(pos.long()[pair.long()], torch.arange(P, device=DEV))
    want = [v for g in range(groups) for r in range(bounds[g], bounds[g + 1], tile_rows) for v in (g, r)]
    assert int(nt) == len(want) // 2 and tl[:len(want)].tolist() == want
    assert bool((tl[len(want):] == -7).all())


@pytest.mark.parametrize("N, D, E, k", [(301, 5120, 16, 1), (70, 96, 8, 2), (1000, 200, 128, 4), (9, 64, 3, 3)])
def test_router_for_many_rows(N, D, E, k):
    """The kernel that shares each router row among eight tokens: the same choices as float64 makes, except
    where two scores tie to within 32-bit rounding; ties still go to the lower expert."""
    h, w = torch.randn(N, D, device=DEV), torch.randn(E, D, device=DEV)
    h[3] = 0.0  # every score of this token ties
    idx, wt = torch.full((N, k), -1, device=DEV, dtype=torch.int32), torch.empty(N, k, device=DEV)
    K().router(h, w, idx, wt, many_rows=True)
    torch.cuda.synchronize()
    scores = h.double() @ w.double().T
    order = torch.sort(scores, dim=-1, descending=True, stable=True)
    chosen = torch.gather(scores, 1, idx.long())
    assert float((order.values[:, :k] - chosen).abs().max()) < 1e-4 * float(scores.abs().max())
    close(wt, torch.sigmoid(chosen), 1e-5)
    assert idx[3].tolist() == list(range(k))
    assert all(len(set(row)) == k for row in idx.tolist())


def test_router_tie_goes_to_the_lower_expert():
    h = torch.zeros(2, 32, device=DEV)
    h[:, 0] = 1
    w = torch.zeros(6, 32, device=DEV)
    w[:, 0] = torch.tensor([0.5, 2.0, 2.0, -1.0, 2.0, 0.0])
    idx, wt = torch.empty(2, 2, device=DEV, dtype=torch.int32), torch.empty(2, 2, device=DEV)
    K().router(h, w, idx, wt)
    assert idx.tolist() == [[1, 2], [1, 2]]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_permute_scale_and_combine(dtype):
    N, D, k, E = 21, 72, 2, 5
    h = torch.randn(N, D, device=DEV)
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(N)]).to(DEV).to(torch.int32)
    wt = torch.rand(N, k, device=DEV)
    off, pair, pos, st = (torch.empty(E + 1, device=DEV, dtype=torch.int32), torch.empty(N * k, device=DEV, dtype=torch.int32),
                          torch.empty(N * k, device=DEV, dtype=torch.int32), status())
    K().expert_sort(idx, off, pair, pos, E, st)
    a = torch.empty(N * k, D, device=DEV, dtype=dtype)
    K().permute_scale(h, pair, wt, a, k)
    ref = (wt.flatten()[pair.long()][:, None] * h[pair.long() // k])
    close(a, ref, 1e-6 if dtype == torch.float32 else 5e-3)
    y, shared, delta = torch.randn(N * k, D, device=DEV), torch.randn(N, D, device=DEV), torch.empty(N, D, device=DEV)
    K().moe_combine(y, shared, pos, delta, k)
    close(delta, shared + y[pos.long()].reshape(N, k, D).sum(1), 1e-6)
    # an appended shared group: offsets get one more entry, rows N*k.. are unscaled copies, the combine adds them
    off2 = torch.empty(E + 2, device=DEV, dtype=torch.int32)
    K().expert_sort(idx, off2, pair, pos, E, st, N)
    assert off2.tolist() == off.tolist() + [N * k + N]
    a2 = torch.empty(N * k + N, D, device=DEV, dtype=dtype)
    K().permute_scale(h, pair, wt, a2, k, N)
    close(a2[: N * k], ref, 1e-6 if dtype == torch.float32 else 5e-3)
    close(a2[N * k:], h, 1e-6 if dtype == torch.float32 else 5e-3)
    y2 = torch.randn(2, N * k + N, D, device=DEV)
    K().moe_combine(y2, None, pos, delta, k, 1, 2, N * k)
    ys = y2.sum(0)
    close(delta, ys[N * k:] + ys[pos.long()].reshape(N, k, D).sum(1), 1e-6)


def test_sampling_argmax_and_draws():
    from tests.plain import llama4_plain as plain

    M, V = 6, 1003
    logits = torch.randn(M, V, device=DEV) * 3
    logits[2, 77] = logits[2, 500] = 50.0  # a tie: the lower index wins
    out = torch.empty(M, device=DEV, dtype=torch.int32)
    K().sample(logits, out)
    want = logits.argmax(-1).tolist()
    want[2] = 77
    assert out.tolist() == want
    temps = torch.tensor([0.0, 0.8, 0.8, 1.5, 0.3, 0.8], device=DEV)
    ks = torch.tensor([0, 0, 16, 64, 5, 1], device=DEV, dtype=torch.int32)
    streams = torch.tensor([3, 3, 9, 2 ** 40 + 5, 0, 7], device=DEV, dtype=torch.int64)
    for step in range(12):
        counters = torch.full((M,), step, device=DEV, dtype=torch.int64)
        K().sample(logits, out, temps, ks, streams, counters, seed=1234)
        got = out.tolist()
        for m in range(M):
            s, c = int(streams[m]), step
            bits = plain.philox4x32((c & 0xFFFFFFFF, c >> 32, s & 0xFFFFFFFF, s >> 32), (1234, 0))
            u = plain.uniform_from_bits(bits[0])
            ref = plain.sample_top(logits[m].cpu(), float(temps[m]), int(ks[m]), u)
            if got[m] != ref:  # allowed only when u sits on the boundary between the two tokens (float32 vs float64 sums)
                p = torch.softmax(logits[m].double().cpu() / float(temps[m]), -1)
                assert abs(got[m] - ref) >= 1 and min(float(p[got[m]]), float(p[ref])) > 0
                us = [plain.sample_top(logits[m].cpu(), float(temps[m]), int(ks[m]), min(max(u + d, 0.0), 0.999999)) for d in (-2e-6, 2e-6)]
                assert got[m] in us, (m, step, got[m], ref)
    # draws follow the distribution: 4000 draws over 3 tokens
    small = torch.tensor([[2.0, 1.0, 0.0]], device=DEV)
    n = 4000
    big = small.expand(n, 3).contiguous()
    o = torch.empty(n, device=DEV, dtype=torch.int32)
    K().sample(big, o, torch.ones(n, device=DEV), torch.zeros(n, device=DEV, dtype=torch.int32),
               torch.arange(n, device=DEV, dtype=torch.int64), torch.zeros(n, device=DEV, dtype=torch.int64), seed=5)
    freq = torch.bincount(o.long(), minlength=3).float() / n
    assert (freq - torch.softmax(small[0], -1)).abs().max() < 0.03


@pytest.mark.parametrize("Hq, Hkv, dh, page, chunk, window, temp", [
    (40, 8, 128, 64, 0, 0, False), (6, 2, 64, 16, 512, 0, False), (16, 1, 128, 32, 0, 300, True), (4, 4, 64, 128, 0, 0, True),
    (10, 2, 128, 16, 1024, 0, False)])
def test_attention_decode_mma(Hq, Hkv, dh, page, chunk, window, temp):
    lens = [1500, 257, 1, 256, 1024, 63]
    q, pages, bt, req, pos, ks, vs = _paged_case(torch.bfloat16, Hq, Hkv, dh, page, lens, [1] * len(lens))
    out, st = torch.empty_like(q), status()
    attn_scale, floor_scale = (0.1, 256.0) if temp else (0.0, 1.0)
    api = K()
    assert api.attention_mma_supported(q.dtype, Hq, Hkv, dh, True)
    for pairs in (len(lens) * Hkv, 4000):  # few pairs: short splits; many pairs: one long split each
        keys, splits = api.attention_decode_plan(max(lens), chunk, window, pairs)
        n = q.shape[0] * Hq * splits
        part_o, part_ml = torch.empty(n * dh, device=DEV), torch.empty(n * 2, device=DEV)
        out.fill_(float("nan"))
        api.attention_decode(q, pages, bt, req, pos, out, dh ** -0.5, chunk, window, attn_scale, floor_scale, part_o, part_ml,
                             splits, keys, st)
        assert int(st) == 0
        for r in range(len(lens)):
            ref = _attention_ref(q[r:r + 1], ks[r], vs[r], pos[r:r + 1].long(), chunk, window, dh ** -0.5, attn_scale, floor_scale)
            close(out[r:r + 1], ref, 1.5e-2)
        # some of the rows only, by a list (the decoded tokens of a step that also holds prompt portions): the
        # same results in those rows, the others untouched
        rows = torch.tensor([4, 0, 3], device=DEV, dtype=torch.int32)
        out2 = torch.full_like(out, 7.0)
        api.attention_decode(q, pages, bt, req, pos, out2, dh ** -0.5, chunk, window, attn_scale, floor_scale, part_o, part_ml,
                             splits, keys, st, rows, 3)
        assert int(st) == 0
        assert torch.equal(out2[rows.long()], out[rows.long()])
        assert bool((out2[[1, 2, 5]] == 7.0).all())


@pytest.mark.parametrize("Hq, Hkv, dh, page, chunk, window, temp", [
    (40, 8, 128, 64, 0, 0, False), (6, 2, 64, 16, 100, 0, False), (8, 1, 128, 32, 0, 70, True), (4, 4, 64, 128, 0, 0, True),
    (10, 2, 128, 16, 64, 0, False)])
def test_attention_prefill_mma(Hq, Hkv, dh, page, chunk, window, temp):
    lens, q_lens = [300, 37, 1, 129, 64], [300, 5, 1, 17, 33]
    q, pages, bt, req, pos, ks, vs = _paged_case(torch.bfloat16, Hq, Hkv, dh, page, lens, q_lens)
    out, st = torch.full_like(q, float("nan")), status()
    attn_scale, floor_scale = (0.1, 64.0) if temp else (0.0, 1.0)
    api = K()
    assert api.attention_mma_supported(q.dtype, Hq, Hkv, dh, False)
    tiles, at = [], 0
    for n in q_lens:
        tiles += [(at + t, min(16, n - t)) for t in range(0, n, 16)]
        at += n
    tl = torch.tensor(tiles, device=DEV, dtype=torch.int32)
    api.attention_prefill(q, pages, bt, req, pos, out, tl, len(tiles), dh ** -0.5, chunk, window, attn_scale, floor_scale, st)
    assert int(st) == 0
    at = 0
    for r, n in enumerate(q_lens):
        ref = _attention_ref(q[at:at + n], ks[r], vs[r], pos[at:at + n].long(), chunk, window, dh ** -0.5, attn_scale, floor_scale)
        close(out[at:at + n], ref, 1.5e-2)
        at += n


def test_mma_attention_finds_one_far_key():
    Hq, Hkv, dh, page = 10, 2, 128, 64
    api = K()
    for far in (0, 63, 64, 255, 256, 257, 1000, 1999):
        q, pages, bt, req, pos, ks, vs = _paged_case(torch.bfloat16, Hq, Hkv, dh, page, [2000], [1], seed=far)
        pg, slot = int(bt[0, far // page]), far % page
        pages[pg, 0, :, slot] = 0
        pages[pg, 0, :, slot, 0] = 40.0
        q[:] = 0
        q[..., 0] = 40.0
        want = pages[pg, 1, :, slot].float().repeat_interleave(Hq // Hkv, 0)
        out, st = torch.empty_like(q), status()
        keys, splits = api.attention_decode_plan(2000, 0, 0, Hkv)
        part_o, part_ml = torch.empty(Hq * splits * dh, device=DEV), torch.empty(Hq * splits * 2, device=DEV)
        api.attention_decode(q, pages, bt, req, pos, out, dh ** -0.5, 0, 0, 0.0, 1.0, part_o, part_ml, splits, keys, st)
        close(out[0], want, 1e-2)
        out2 = torch.empty_like(q)
        api.attention_prefill(q, pages, bt, req, pos, out2, torch.tensor([[0, 1]], device=DEV, dtype=torch.int32), 1,
                              dh ** -0.5, 0, 0, 0.0, 1.0, st)
        close(out2[0], want, 1e-2)


def test_gemm_stream_partials_and_swiglu_epilogue():
    from jax_llm_examples_b200.parts.linear import interleave_gate_up

    api = K()
    M, N, Kd = 9, 256, 2048
    a, w = torch.randn(M, Kd, device=DEV).bfloat16(), torch.randn(N, Kd, device=DEV).bfloat16()
    parts, st = torch.full((4, M, N), float("nan"), device=DEV), status()
    used = api.gemm_stream(a, w, parts, st, splits=4, mode=api.GEMM_PARTIALS)
    assert used == 4 and int(st) == 0
    close(parts.sum(0), a.double() @ w.double().T, 1e-5)
    # SwiGLU epilogue on interleaved rows, dense and grouped
    F = 160
    wgu = (torch.randn(2 * F, Kd, device=DEV) * 0.05).bfloat16()
    act = torch.full((M, F), float("nan"), device=DEV, dtype=torch.bfloat16)
    api.gemm_stream(a, interleave_gate_up(wgu), act, st, mode=api.GEMM_SWIGLU)
    g, u = a.double() @ wgu[:F].double().T, a.double() @ wgu[F:].double().T
    close(act, torch.nn.functional.silu(g) * u, 1e-2)
    E, rows = 5, 70
    a2 = torch.randn(rows, Kd, device=DEV).bfloat16()
    we = (torch.randn(E, 2 * F, Kd, device=DEV) * 0.05).bfloat16()
    off = _groups(E, 3, rows)
    act2 = torch.full((rows, F), float("nan"), device=DEV)
    api.gemm_stream(a2, interleave_gate_up(we), act2, st, offsets=off.to(DEV), rows_hint=20, mode=api.GEMM_SWIGLU)
    assert int(st) == 0
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            g, u = a2[lo:hi].double() @ we[e, :F].double().T, a2[lo:hi].double() @ we[e, F:].double().T
            close(act2[lo:hi], torch.nn.functional.silu(g) * u, 1e-4)
    # wide token tiles and outputs in multiples of 256: the paired kernel's epilogue
    E, rows, F2 = 3, 400, 256
    a3 = torch.randn(rows, Kd, device=DEV).bfloat16()
    we3 = (torch.randn(E, 2 * F2, Kd, device=DEV) * 0.05).bfloat16()
    off = _groups(E, 5, rows)
    act3 = torch.full((rows, F2), float("nan"), device=DEV, dtype=torch.bfloat16)
    api.gemm_stream(a3, interleave_gate_up(we3), act3, st, offsets=off.to(DEV), rows_hint=160, mode=api.GEMM_SWIGLU)
    assert int(st) == 0
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            g, u = a3[lo:hi].double() @ we3[e, :F2].double().T, a3[lo:hi].double() @ we3[e, F2:].double().T
            close(act3[lo:hi], torch.nn.functional.silu(g) * u, 1e-2)
    # the activation kernel reads the same interleaved layout and split partials
    gu = torch.randn(3, 7, 2 * F, device=DEV)
    out = torch.empty(7, F, device=DEV)
    api.silu_mul(interleave_gate_up(gu.transpose(1, 2)).transpose(1, 2).contiguous(), out, splits=3, interleaved=True)
    s = gu.sum(0)
    close(out, torch.nn.functional.silu(s[:, :F]) * s[:, F:], 1e-5)


def test_add_rmsnorm_with_partials_and_fused_router():
    N, D, E, k, eps = 19, 1000, 12, 3, 1e-5
    x, parts, g = torch.randn(N, D, device=DEV), torch.randn(3, N, D, device=DEV), 1 + 0.1 * torch.randn(D, device=DEV)
    w = torch.randn(E, D, device=DEV)
    s = x + parts[0] + parts[1] + parts[2]
    ref = g * s / torch.sqrt((s * s).mean(-1, keepdim=True) + eps)
    xc, out, out32 = x.clone(), torch.empty(N, D, device=DEV, dtype=torch.bfloat16), torch.empty(N, D, device=DEV)
    idx, wt = torch.empty(N, k, device=DEV, dtype=torch.int32), torch.empty(N, k, device=DEV)
    K().add_rmsnorm(xc, parts, g, eps, out, out32, None, 3, w, idx, wt)
    close(out32, ref, 2e-6), close(out, ref, 5e-3)
    assert torch.allclose(xc, s, atol=1e-6)
    scores = out32.double() @ w.double().T
    order = torch.sort(scores, dim=-1, descending=True, stable=True)
    assert torch.equal(idx.long(), order.indices[:, :k])
    close(wt, torch.sigmoid(order.values[:, :k]), 1e-5)


@pytest.mark.parametrize("want32", [False, True])
@pytest.mark.parametrize("N, D, E, k, splits", [(5, 5120, 16, 1, 3), (1, 1288, 5, 2, 1), (32, 2048, 128, 4, 2)])
def test_add_rmsnorm_router_on_few_rows_by_a_cluster(N, D, E, k, splits, want32):
    """A few rows, bfloat16 output, a router and no 32-bit copy: eight blocks share a row (a cluster with
    distributed shared memory).  The same sums in another order: compare with float64."""
    eps = 1e-5
    x, parts, g = torch.randn(N, D, device=DEV), torch.randn(splits, N, D, device=DEV), 1 + 0.1 * torch.randn(D, device=DEV)
    w = torch.randn(E, D, device=DEV)
    s = x.double() + parts.double().sum(0)
    ref = g.double() * s / torch.sqrt((s * s).mean(-1, keepdim=True) + eps)
    xc, out = x.clone(), torch.full((N, D), float("nan"), device=DEV, dtype=torch.bfloat16)
    idx, wt = torch.full((N, k), -1, device=DEV, dtype=torch.int32), torch.empty(N, k, device=DEV)
    out32 = torch.full((N, D), float("nan"), device=DEV) if want32 else None
    K().add_rmsnorm(xc, parts, g, eps, out, out32, None, splits, w, idx, wt)
    torch.cuda.synchronize()
    close(out, ref, 5e-3)
    if want32:
        close(out32, ref, 2e-6)
    assert torch.allclose(xc.double(), s, atol=1e-5)
    scores = ref @ w.double().T
    order = torch.sort(scores, dim=-1, descending=True, stable=True)
    # a choice may differ from float64's only where two scores tie to within 32-bit rounding
    chosen = torch.gather(scores, 1, idx.long())
    assert float((order.values[:, :k] - chosen).abs().max()) < 1e-3 * float(scores.abs().max())
    close(wt, torch.sigmoid(chosen), 1e-4)


@pytest.mark.parametrize("N,D,E,k,extra,tile_rows", [(1, 1024, 16, 1, 1, 16), (1, 1280, 4, 2, 0, 0), (5, 1024, 16, 1, 0, 16),
                                                      (16, 2048, 40, 2, 16, 32), (3, 1024, 130, 4, 3, 16)])
def test_add_rmsnorm_router_that_also_sorts_and_gathers(N, D, E, k, extra, tile_rows):
    """A decode step's norm + router kernel can do what expert_sort and permute_scale would do next (one launch for
    three).  Its sort and its gathered rows must be exactly theirs, from the same choices; launch after launch (the
    ticket counter returns to zero)."""
    from types import SimpleNamespace

    eps, P = 1e-5, N * k
    g, w = 1 + 0.1 * torch.randn(D, device=DEV), torch.randn(E, D, device=DEV)
    counter, st = torch.zeros(1, device=DEV, dtype=torch.int32), status()
    groups = E + (extra > 0)
    for launch in range(3):
        x, parts = torch.randn(N, D, device=DEV), torch.randn(2, N, D, device=DEV)
        out, out32 = torch.empty(N, D, device=DEV, dtype=torch.bfloat16), torch.empty(N, D, device=DEV)
        idx, wt = torch.full((N, k), -1, device=DEV, dtype=torch.int32), torch.empty(N, k, device=DEV)
        tiles = (torch.full((2 * (-(-(P + extra) // tile_rows) + groups),), -7, device=DEV, dtype=torch.int32),
                 torch.full((1,), -7, device=DEV, dtype=torch.int32)) if tile_rows else None
        d = SimpleNamespace(counter=counter, offsets=torch.full((E + 2,), -7, device=DEV, dtype=torch.int32),
                            sorted_pair=torch.full((P,), -7, device=DEV, dtype=torch.int32),
                            sorted_pos=torch.full((P,), -7, device=DEV, dtype=torch.int32), tiles=tiles,
                            a_sorted=torch.full((P + extra, D), float("nan"), device=DEV, dtype=torch.bfloat16),
                            extra_rows=extra, tile_rows=tile_rows, status=st)
        assert K().add_rmsnorm(x, parts, g, eps, out, out32, None, 2, w, idx, wt, d)
        torch.cuda.synchronize()
        assert int(counter) == 0 and int(st) == 0
        # the separate kernels, from the same choices and the same normed rows
        offsets, pair, pos = (torch.full_like(t, -9) for t in (d.offsets, d.sorted_pair, d.sorted_pos))
        tiles2 = tuple(torch.full_like(t, -9) for t in tiles) if tiles else ()
        K().expert_sort(idx, offsets, pair, pos, E, st, extra, tile_rows, *tiles2)
        a2 = torch.empty_like(d.a_sorted)
        K().permute_scale(out32, pair, wt, a2, k, extra)
        torch.cuda.synchronize()
        n_off = E + 2 if extra else E + 1
        assert torch.equal(d.offsets[:n_off], offsets[:n_off]) and torch.equal(d.sorted_pair, pair) and torch.equal(d.sorted_pos, pos)
        if tiles:
            nt = int(tiles2[1])
            assert int(tiles[1]) == nt and torch.equal(tiles[0][:2 * nt], tiles2[0][:2 * nt])
            # nothing is written past the list (a lane of the scan beyond the last group once listed tiles of its own)
            assert bool((tiles[0][2 * nt:] == -7).all()) and bool((tiles2[0][2 * nt:] == -9).all())
        assert torch.equal(d.a_sorted, a2)


def test_rope_kv_store_from_float32_partials():
    N, Hq, Hkv, dh, page, P, eps = 5, 4, 2, 64, 16, 4, 1e-5
    parts = torch.randn(2, N, (Hq + 2 * Hkv) * dh, device=DEV)
    pos = torch.arange(7, 7 + N, device=DEV, dtype=torch.int32)
    req = torch.zeros(N, device=DEV, dtype=torch.int32)
    bt = torch.tensor([[2, 0, 3, 1]], device=DEV, dtype=torch.int32)
    pages = torch.zeros(P, 2, Hkv, page, dh, device=DEV, dtype=torch.bfloat16)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, dh, 2, device=DEV).float() / dh))
    q_out, st = torch.empty(N, Hq, dh, device=DEV, dtype=torch.bfloat16), status()
    K().rope_kv_store(parts, q_out, pages, bt, req, pos, inv_freq, True, eps, Hq, Hkv, dh, st, splits=2)
    x = parts.sum(0).reshape(N, Hq + 2 * Hkv, dh)
    q = _rope_ref(x[:, :Hq], pos, inv_freq)
    q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps)
    close(q_out, q, 8e-3)
    v = x[:, Hq + Hkv:]
    for n in range(N):
        pg, slot = int(bt[0, int(pos[n]) // page]), int(pos[n]) % page
        close(pages[pg, 1, :, slot], v[n], 8e-3)


def test_two_stage_argmax():
    M, V = 7, 202048
    logits = torch.randn(M, V, device=DEV)
    logits[3, 5000] = logits[3, 150000] = 99.0
    logits[5, V - 1] = 100.0
    out = torch.empty(M, device=DEV, dtype=torch.int32)
    K().argmax(logits, out, torch.empty(32 * M, device=DEV), torch.empty(32 * M, device=DEV, dtype=torch.int32))
    want = logits.argmax(-1).tolist()
    want[3] = 5000
    assert out.tolist() == want


def test_gemm_stream_grouped_split_k_partials():
    api = K()
    E, rows, N, Kd = 4, 5, 256, 2048
    a, w = torch.randn(rows, Kd, device=DEV).bfloat16(), torch.randn(E, N, Kd, device=DEV).bfloat16()
    off = torch.tensor([0, 2, 2, 4, 5], device=DEV, dtype=torch.int32)
    parts, st = torch.full((4, rows, N), float("nan"), device=DEV), status()
    used = api.gemm_stream(a, w, parts, st, offsets=off, rows_hint=2, splits=4, mode=api.GEMM_PARTIALS)
    assert used == 4 and int(st) == 0
    got = parts.sum(0)
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            close(got[lo:hi], a[lo:hi].double() @ w[e].double().T, 1e-5)


@pytest.mark.parametrize("E, N, k, extra", [(128, 300, 1, 0), (16, 40, 2, 40), (5, 7, 1, 7)])
def test_grouped_product_with_the_sort_kernels_tile_list(E, N, k, extra):
    """expert_sort lists the row tiles that hold rows; the grouped product then finds its work from that list."""
    api = K()
    D, Nout = 128, 256
    idx = torch.randint(0, E, (N, k), device=DEV, dtype=torch.int32)
    groups, rows = E + (extra > 0), N * k + extra
    hint = max(3, extra)
    tile_rows = api.gemm_stream_token_tile(hint)
    off = torch.empty(E + 2, device=DEV, dtype=torch.int32)
    pair, pos, st = torch.empty(N * k, device=DEV, dtype=torch.int32), torch.empty(N * k, device=DEV, dtype=torch.int32), status()
    tl = torch.full((2 * (-(-rows // tile_rows) + groups),), -1, device=DEV, dtype=torch.int32)
    nt = torch.zeros(1, device=DEV, dtype=torch.int32)
    api.expert_sort(idx, off, pair, pos, E, st, extra, tile_rows, tl, nt)
    offs = off[: groups + 1].tolist()
    want = [(e, r) for e in range(groups) for r in range(offs[e], offs[e + 1], tile_rows)]
    assert int(nt) == len(want) and tl[: 2 * len(want)].view(-1, 2).tolist() == [list(t) for t in want]
    a = torch.randn(rows, D, device=DEV).bfloat16()
    w = torch.randn(groups, Nout, D, device=DEV).bfloat16()
    out = torch.full((rows, Nout), float("nan"), device=DEV)
    api.gemm_stream(a, w, out, st, offsets=off[: groups + 1].contiguous(), rows_hint=hint, tiles=(tl, nt))
    assert int(st) == 0
    for e in range(groups):
        lo, hi = offs[e], offs[e + 1]
        if hi > lo:
            close(out[lo:hi], a[lo:hi].double() @ w[e].double().T, 1e-5)


@pytest.mark.parametrize("E, N, k, extra", [(16, 1, 1, 1), (16, 8, 1, 0), (40, 30, 2, 0)])
def test_a_grouped_product_right_after_another_over_the_same_groups(E, N, k, extra):
    """An expert layer's down product follows its gate/up product over the same offsets and tile list; told so, it
    finds its tile and asks for its weights before it waits for the gate/up product.  The result is the one of the
    product that waits first, every time (the pair is launched back to back, programmatic dependent launch and all)."""
    api = K()
    D, F = 256, 512
    idx = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(N)]).to(torch.int32)
    groups, rows = E + (extra > 0), N * k + extra
    hint = max(3, extra)
    tile_rows = api.gemm_stream_token_tile(hint)
    off = torch.empty(E + 2, device=DEV, dtype=torch.int32)
    pair, pos, st = torch.empty(N * k, device=DEV, dtype=torch.int32), torch.empty(N * k, device=DEV, dtype=torch.int32), status()
    tl = torch.full((2 * (-(-rows // tile_rows) + groups),), -1, device=DEV, dtype=torch.int32)
    nt = torch.zeros(1, device=DEV, dtype=torch.int32)
    a = torch.randn(rows, D, device=DEV).bfloat16()
    w_gu = (0.1 * torch.randn(groups, 2 * F, D, device=DEV)).bfloat16()
    w_dn = (0.1 * torch.randn(groups, D, F, device=DEV)).bfloat16()
    offs = off[: groups + 1]
    results = []
    for settled in (False, True, True, True):
        act = torch.full((rows, F), float("nan"), device=DEV, dtype=torch.bfloat16)
        y = torch.full((2, rows, D), float("nan"), device=DEV)
        api.expert_sort(idx, off, pair, pos, E, st, extra, tile_rows, tl, nt)
        api.gemm_stream(a, w_gu, act, st, offsets=offs, rows_hint=hint, mode=api.GEMM_SWIGLU, tiles=(tl, nt))
        used = api.gemm_stream(act, w_dn, y, st, offsets=offs, rows_hint=hint, splits=2, mode=api.GEMM_PARTIALS, tiles=(tl, nt),
                               offsets_settled=settled)
        results.append(y[:used].sum(0))
    torch.cuda.synchronize()
    assert int(st) == 0 and not bool(torch.isnan(results[0]).any())
    for r in results[1:]:
        assert torch.equal(r, results[0])


@pytest.mark.parametrize("kind, size", [("window", 100), ("chunk", 192), ("chunk", 80)])
def test_attention_edges_of_windows_and_chunks(kind, size):
    """A key whose score would swamp all others sits exactly on the first position a query may see, and then
    one position before it: seen, the output is that key's value; one before, the output must not contain
    it at all.  Random keys would hide an edge that is off by one.  All three kernels, 32-bit and bfloat16."""
    Hq, Hkv, dh, page = 6, 2, 64, 16
    api = K()
    L = 500
    p = L - 1
    first = p - size + 1 if kind == "window" else (p // size) * size
    chunk, window = (size, 0) if kind == "chunk" else (0, size)
    for dtype in (torch.float32, torch.bfloat16):
        for hot, seen in ((first, True), (first - 1, False)):
            q, pages, bt, req, pos, ks, vs = _paged_case(dtype, Hq, Hkv, dh, page, [L], [1], seed=hot)
            pg, slot = int(bt[0, hot // page]), hot % page
            pages[pg, 0, :, slot] = 0
            pages[pg, 0, :, slot, 0] = 40.0
            pages[pg, 1, :, slot] = 1000.0  # its value is unmistakable
            q[:] = 0
            q[..., 0] = 40.0
            outs = []
            out, st = torch.empty_like(q), status()
            api.attention_generic(q, pages, bt, req, pos, out, dh ** -0.5, chunk, window, 0.0, 1.0, st)
            outs.append(out)
            if dtype == torch.bfloat16:
                keys, splits = api.attention_decode_plan(L, chunk, window, Hkv)
                part_o, part_ml = torch.empty(Hq * splits * dh, device=DEV), torch.empty(Hq * splits * 2, device=DEV)
                o2 = torch.empty_like(q)
                api.attention_decode(q, pages, bt, req, pos, o2, dh ** -0.5, chunk, window, 0.0, 1.0, part_o, part_ml, splits, keys, st)
                o3 = torch.empty_like(q)
                api.attention_prefill(q, pages, bt, req, pos, o3, torch.tensor([[0, 1]], device=DEV, dtype=torch.int32), 1,
                                      dh ** -0.5, chunk, window, 0.0, 1.0, st)
                outs += [o2, o3]
            assert int(st) == 0
            for o in outs:
                if seen:
                    assert float((o.float() - 1000.0).abs().max()) < 10.0
                else:
                    assert float(o.float().abs().max()) < 10.0  # ordinary values are ~N(0, 1)


@pytest.mark.parametrize("Hq, Hkv, page, chunk, window, temp", [
    (4, 2, 64, 0, 0, False), (10, 2, 128, 0, 0, True), (3, 1, 64, 200, 0, False), (4, 4, 64, 0, 150, False),
    (2, 1, 64, 128, 0, False)])
def test_attention_prefill_tc(Hq, Hkv, page, chunk, window, temp):
    """The tcgen05 flash kernel: tiles of up to 128 tokens, several requests, cached history before the portion."""
    dh = 128
    lens, q_lens = [700, 128, 130, 300], [700, 128, 1, 45]
    q, pages, bt, req, pos, ks, vs = _paged_case(torch.bfloat16, Hq, Hkv, dh, page, lens, q_lens)
    out, st = torch.full_like(q, float("nan")), status()
    attn_scale, floor_scale = (0.1, 64.0) if temp else (0.0, 1.0)
    api = K()
    assert api.attention_prefill_tc_supported(q.dtype, Hq, Hkv, dh, page)
    tiles, at = [], 0
    for n in q_lens:
        tiles += [(at + t, min(128, n - t)) for t in range(0, n, 128)]
        at += n
    tl = torch.tensor(tiles, device=DEV, dtype=torch.int32)
    api.attention_prefill_tc(q, pages, bt, req, pos, out, tl, len(tiles), dh ** -0.5, chunk, window, attn_scale, floor_scale, st)
    torch.cuda.synchronize()
    assert int(st) == 0
    at = 0
    for r, n in enumerate(q_lens):
        ref = _attention_ref(q[at:at + n], ks[r], vs[r], pos[at:at + n].long(), chunk, window, dh ** -0.5, attn_scale, floor_scale)
        close(out[at:at + n], ref, 1.5e-2)
        at += n


@pytest.mark.parametrize("out_dtype, tol", [(torch.float32, 2e-6), (torch.bfloat16, 5e-3)])
@pytest.mark.parametrize("N, D, k, E", [(5, 5120, 1, 16), (70, 200, 2, 8), (3, 1030, 3, 4)])
def test_add_rmsnorm_adds_a_sum_of_terms_with_gathered_rows(out_dtype, tol, N, D, k, E):
    """The norm adds an expert layer's output while it is still in expert order: a plain term with split-K partials
    (a shared expert), a term at a row offset (a shared expert riding as the last group), and a term whose k rows per
    token are gathered by an index; in that order, as the combine kernel would."""
    g = torch.Generator(device=DEV).manual_seed(N)
    x = torch.randn(N, D, device=DEV, generator=g)
    gamma = 1 + 0.1 * torch.randn(D, device=DEV, generator=g)
    shared = torch.randn(2, N, D, device=DEV, generator=g)
    rows = N * k + N
    y = torch.randn(3, rows, D, device=DEV, generator=g)
    pos = torch.randperm(N * k, device=DEV).to(torch.int32)  # sorted row of each (token, choice) pair
    terms = [(shared, 2, None, 1, 0), (y, 3, None, 1, N * k), (y, 3, pos, k, 0)]
    ref = x + shared.sum(0) + y.sum(0)[N * k:] + y.sum(0)[pos.long()].reshape(N, k, D).sum(1)
    want = gamma * ref / torch.sqrt((ref * ref).mean(-1, keepdim=True) + 1e-5)
    out = torch.empty(N, D, device=DEV, dtype=out_dtype)
    out32 = torch.empty(N, D, device=DEV)
    x1 = x.clone()
    K().add_rmsnorm(x1, terms, gamma, 1e-5, out, out32)
    close(x1, ref, 2e-6)
    close(out, want, tol)
    close(out32, want, 2e-6)
    # the wanted rows only (the final norm): x is left alone
    idx = torch.tensor([N - 1, 0], device=DEV, dtype=torch.int32)
    x2, out2 = x.clone(), torch.empty(2, D, device=DEV, dtype=out_dtype)
    K().add_rmsnorm(x2, terms, gamma, 1e-5, out2, None, idx)
    assert torch.equal(x2, x)
    close(out2, want[idx.long()], tol)
    # with the router in the same kernel (a cluster of blocks per row for few wide rows in bfloat16)
    w_router = torch.randn(E, D, device=DEV, generator=g)
    ti, tw = torch.empty(N, 1, device=DEV, dtype=torch.int32), torch.empty(N, 1, device=DEV)
    x3 = x.clone()
    K().add_rmsnorm(x3, terms, gamma, 1e-5, out, out32, None, 1, w_router, ti, tw)
    close(x3, ref, 2e-6)
    close(out32, want, 2e-6)
    scores = want @ w_router.T
    chosen = torch.gather(scores, 1, ti.long())
    assert float((scores.max(-1, keepdim=True).values - chosen).max()) < 1e-3 * float(scores.abs().max())
