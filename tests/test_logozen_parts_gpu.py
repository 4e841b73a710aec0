"""Each mechanism of Logozen alone: the kernel behind it against the plain function, on inputs made so that a fault shows."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_logozen as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from mini_engine_b200 import ops
    ops.require_extension()
    return ops


def _meta(lens, contexts):
    """Step metadata as the kernels read it: requests that bring one token come first."""
    assert all(n == 1 for n in lens[:sum(1 for n in lens if n == 1)])
    cu = np.concatenate(([0], np.cumsum(lens))).astype(np.int32)
    D = sum(1 for n in lens if n == 1)
    token_req = torch.tensor(np.repeat(np.arange(len(lens)), lens), dtype=torch.int32, device=DEV)
    lists = {}
    for tq in (8, 16, 32, 64):
        tiles = [(b, q0) for b in range(D, len(lens)) for q0 in range(0, lens[b], tq)]
        lists[tq] = (torch.tensor(tiles or [(0, 0)], dtype=torch.int32, device=DEV), len(tiles))
    return SimpleNamespace(cu_seqlens=torch.tensor(cu, device=DEV), context_lens=torch.tensor(contexts, dtype=torch.int32, device=DEV),
                           num_reqs=len(lens), num_decodes=D, tile_lists=lists, token_req=token_req, max_context_len=max(contexts),
                           workspace=lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=DEV))


def g(seed):
    return torch.Generator().manual_seed(seed)


# ---- residual streams and the layer norm ---------------------------------------------------------------
@pytest.mark.parametrize("S, W", [(1, 40), (3, 48), (8, 300), (4, 1030), (13, 36)])
def test_stream_update_mix_in_and_layer_norm(S, W):
    ops = _ops()
    T, eps = 7, 1e-5
    x = torch.randn(S, T, W, generator=g(S)) * 3 + 0.5
    y = torch.randn(T, W, generator=g(1))
    mix = torch.eye(S) + 0.2 * torch.randn(S, S, generator=g(2))
    outw, inw, nw = torch.rand(S, generator=g(3)) + 0.5, torch.rand(S, generator=g(4)), torch.rand(W, generator=g(5)) + 0.5
    new = torch.einsum("sr,stw->rtw", mix.double(), x.double()) + outw.double()[:, None, None] * y.double()[None]
    ref = plain.layer_norm(torch.einsum("s,stw->tw", inw.double(), new), nw.double(), eps)
    xd, out = x.to(DEV), torch.empty(T, W, device=DEV)
    ops.hc_norm(xd, update=(y.to(DEV), mix.to(DEV).contiguous(), outw.to(DEV)), mix_in=inw.to(DEV), norm_weight=nw.to(DEV), eps=eps, out=out)
    assert torch.allclose(xd.cpu().double(), new, atol=1e-5)
    assert torch.allclose(out.cpu().double(), ref, atol=2e-5)
    # the sum of the streams at two rows, with a pending update, writes nothing
    xd2, rows = x.to(DEV), torch.tensor([5, 2], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, W, device=DEV, dtype=torch.bfloat16)
    ops.hc_norm(xd2, update=(y.to(DEV).bfloat16(), mix.to(DEV).contiguous(), outw.to(DEV)), norm_weight=nw.to(DEV), eps=eps, out=out2, rows=rows)
    new2 = torch.einsum("sr,stw->rtw", mix.double(), x.double()) + outw.double()[:, None, None] * y.bfloat16().double()[None]
    ref2 = plain.layer_norm(new2.sum(0), nw.double(), eps)[[5, 2]]
    assert torch.equal(xd2.cpu(), x)
    assert torch.allclose(out2.cpu().double(), ref2, atol=3e-2, rtol=1e-2)


def test_layer_norm_subtracts_the_mean():
    """A constant offset must not change the result (an RMS norm in its place would)."""
    ops = _ops()
    W = 64
    x = torch.randn(1, 3, W, generator=g(0))
    nw = torch.ones(W)
    a, b = torch.empty(3, W, device=DEV), torch.empty(3, W, device=DEV)
    ops.hc_norm(x.to(DEV), norm_weight=nw.to(DEV), eps=1e-6, out=a)
    ops.hc_norm((x + 100.0).to(DEV), norm_weight=nw.to(DEV), eps=1e-6, out=b)
    assert torch.allclose(a, b, atol=2e-4)


# ---- short convolution with state ----------------------------------------------------------------------
@pytest.mark.parametrize("taps", [1, 2, 3, 5])
def test_short_convolution_in_portions_with_slots_used_again(taps):
    ops = _ops()
    W, slots = 70, 3
    seqs = [torch.randn(n, W, generator=g(10 + n)) for n in (23, 9, 31)]
    wt = torch.randn(W, taps, generator=g(1)) * 0.5
    ref = [plain.causal_conv_residual(s.double(), wt.double()) for s in seqs]
    state = torch.full((slots, max(taps - 1, 1), W), float("nan"), device=DEV)[:, :taps - 1].contiguous()   # what a request before left
    slot_of = [2, 0, 2]                                     # request 2 takes request 0's slot once that has ended
    got = [[] for _ in seqs]
    # steps: (request, tokens) pairs; one token comes first in a batch; portions of 1, 2 and more, shorter than taps too
    plan = [[(1, 1), (0, 5)], [(0, 1), (1, 2)], [(1, 1), (0, 2)], [(0, 1), (1, 5)], [(0, 14)], [(2, 2)], [(2, 1)], [(2, 1)], [(2, 27)]]
    pos = [0, 0, 0]
    for step in plan:
        lens = [n for _, n in step]
        h = torch.cat([seqs[r][pos[r]:pos[r] + n] for r, n in step]).to(DEV)
        meta = _meta(lens, [pos[r] + n for r, n in step])
        out = torch.empty_like(h)
        ops.short_conv(h, wt.to(DEV), state if taps > 1 else None, meta.token_req, meta,
                       torch.tensor([slot_of[r] for r, _ in step], dtype=torch.int32, device=DEV), out)
        o = 0
        for r, n in step:
            got[r].append(out[o:o + n].cpu())
            o += n
            pos[r] += n
    for r in (0, 2):
        assert pos[r] == len(seqs[r])
        assert torch.allclose(torch.cat(got[r]).double(), ref[r], atol=1e-5), f"request {r}"
    assert torch.allclose(torch.cat(got[1]).double(), ref[1][:pos[1]], atol=1e-5)


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_norm_and_convolution_in_one_kernel_for_single_tokens(taps):
    """Two requests token by token (the second starts later, in a slot that holds another request's leftovers): layer norm of
    the mixed streams, then h + conv(h) with the state moved on, against the plain functions on the whole sequences."""
    ops = _ops()
    S, W, eps, n = 3, 50, 1e-5, 9
    xs = [torch.randn(S, n, W, generator=g(20 + r)) * 2 for r in range(2)]
    inw, nw = torch.rand(S, generator=g(1)) + 0.2, torch.rand(W, generator=g(2)) + 0.5
    wt = torch.randn(W, taps, generator=g(3)) * 0.5
    ref = [plain.causal_conv_residual(plain.layer_norm(torch.einsum("s,stw->tw", inw.double(), x.double()), nw.double(), eps), wt.double())
           for x in xs]
    state = torch.full((4, max(taps - 1, 1), W), float("nan"), device=DEV)[:, :taps - 1].contiguous()
    slots = torch.tensor([3, 1], dtype=torch.int32, device=DEV)
    for t in range(n + 2):
        live = [r for r in range(2) if 0 <= t - 2 * r < n]               # request 1 starts two steps later
        x = torch.stack([xs[r][:, t - 2 * r] for r in live], dim=1).contiguous().to(DEV)          # [S, live, W]
        out = torch.empty(len(live), W, device=DEV)
        lens = torch.tensor([t - 2 * r + 1 for r in live], dtype=torch.int32, device=DEV)
        ops.hc_norm(x, mix_in=inw.to(DEV), norm_weight=nw.to(DEV), eps=eps, out=out,
                    conv=(wt.to(DEV), state if taps > 1 else None, slots[live].contiguous(), lens))
        for k, r in enumerate(live):
            assert torch.allclose(out[k].cpu().double(), ref[r][t - 2 * r], atol=2e-5), f"request {r} token {t - 2 * r}"


# ---- PolyNorm ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("F", [24, 333, 2048])
def test_polynorm(F):
    ops = _ops()
    z = torch.randn(5, F, generator=g(F)) * 2.5
    coef = torch.tensor([0.7, -0.4, 0.9, 0.25])
    a, b, c, e = coef.double()
    zz = z.double()
    ref = a * plain.unit_rms(zz, 1e-5) + b * plain.unit_rms(zz ** 2, 1e-5) + c * plain.unit_rms(zz ** 3, 1e-5) + e
    out = torch.empty(5, F, device=DEV)
    ops.polynorm(z.to(DEV), coef.to(DEV), 1e-5, out)
    assert torch.allclose(out.cpu().double(), ref, atol=2e-5)


# ---- the matrix-memory recurrence -------------------------------------------------------------------------
def _mlstm_case(H, D, V, T, seed, cap=6.0, gate_gain=3.0):
    W = 32
    m = {"heads": H, "dim": D, "vdim": V, "gate_cap": cap}
    w = {"q": torch.randn(H * D, W, generator=g(seed)) * 0.3, "k": torch.randn(H * D, W, generator=g(seed + 1)) * 0.3,
         "v": torch.randn(H * V, W, generator=g(seed + 2)) * 0.3, "g": torch.randn(H * V, W, generator=g(seed + 3)) * 0.3,
         "i": torch.randn(H, W, generator=g(seed + 4)) * gate_gain, "f": torch.randn(H, W, generator=g(seed + 5)) * gate_gain,
         "i.b": torch.randn(H, generator=g(seed + 6)), "f.b": torch.randn(H, generator=g(seed + 7)) + 2,
         "norm": torch.rand(H * V, generator=g(seed + 8)) + 0.5, "o": torch.eye(H * V)}
    h = torch.randn(T, W, generator=g(seed + 9))
    return m, w, h


def _run_mlstm(ops, m, w, h, cuts, slot=1, slots=3, eps=1e-5):
    H, D, V = m["heads"], m["dim"], m["vdim"]
    packed = torch.cat([w[k] for k in ("q", "k", "v", "g", "i", "f")]).to(DEV)
    offs, o = {}, 0
    for k in ("q", "k", "v", "g", "i", "f"):
        offs[k], o = o, o + w[k].shape[0]
    S = torch.full((slots, H, D, V), float("nan"), device=DEV)
    n = torch.full((slots, H, D), float("nan"), device=DEV)
    mm = torch.full((slots, H), float("nan"), device=DEV)
    outs, pos = [], 0
    all_proj = h.to(DEV) @ packed.T                  # once for the whole sequence: a product's rounding may depend on its rows
    for c in cuts:
        proj = all_proj[pos:pos + c].contiguous()
        meta = _meta([c], [pos + c])
        obuf = torch.empty(c, H * V, device=DEV)
        ops.mlstm_scan(proj, offs, w["i.b"].to(DEV), w["f.b"].to(DEV), m["gate_cap"], S, n, mm, meta,
                       torch.tensor([slot], dtype=torch.int32, device=DEV), obuf, H, D, V, D ** -0.5)
        gated = torch.empty(c, H * V, device=DEV)
        ops.mlstm_out(obuf, proj, offs["g"], w["norm"].to(DEV), eps, gated, H, V)
        outs.append(gated.cpu())
        pos += c
    return torch.cat(outs)


@pytest.mark.parametrize("H, D, V", [(2, 16, 32), (3, 24, 40), (1, 72, 8), (2, 8, 100)])
def test_mlstm_against_the_plain_recurrence_and_cut_anywhere(H, D, V):
    ops = _ops()
    T = 200
    m, w, h = _mlstm_case(H, D, V, T, seed=H * 100 + D)
    ref = plain.mlstm(h.double(), {"x." + k: v.double() for k, v in w.items()}, "x.", m, 1e-5)
    whole = _run_mlstm(ops, m, w, h, [T])                              # chunks of 64 tokens and a rest of 8
    assert torch.allclose(whole.double(), ref, atol=3e-4, rtol=1e-3)
    single = _run_mlstm(ops, m, w, h, [1] * T, slot=2)                 # token by token
    assert torch.allclose(single.double(), ref, atol=3e-4, rtol=1e-3)
    cut = _run_mlstm(ops, m, w, h, [2, 1, 30, 2, 64, 1, 65, 35], slot=0)
    assert torch.allclose(cut.double(), ref, atol=3e-4, rtol=1e-3)
    # the state is carried in float32: whole, cut and token by token differ by the order of the sums alone
    assert torch.allclose(whole, single, atol=5e-5, rtol=1e-4) and torch.allclose(whole, cut, atol=5e-5, rtol=1e-4)
    ops.mlstm_chunks = False
    try:                                                                # token by token, a token's arithmetic is the same wherever
        assert torch.equal(_run_mlstm(ops, m, w, h, [T]), single)       # the sequence was cut
    finally:
        ops.mlstm_chunks = True


def test_mlstm_gates_saturate_at_the_cap_and_the_maximum_starts_at_zero():
    """Large gate inputs: without the cap exp() of the input gate would dwarf everything; with a running maximum that
    started at minus infinity the first tokens' denominators would differ."""
    ops = _ops()
    m, w, h = _mlstm_case(2, 16, 32, 40, seed=5, cap=4.0, gate_gain=40.0)
    w["i.b"] = torch.tensor([-30.0, 30.0])
    ref = plain.mlstm(h.double(), {"x." + k: v.double() for k, v in w.items()}, "x.", m, 1e-5)
    got = _run_mlstm(ops, m, w, h, [3, 37])
    assert torch.allclose(got.double(), ref, atol=3e-4, rtol=1e-3)


# ---- attention through a latent ------------------------------------------------------------------------------
def _plain_rows_attention(qa, qr, rows, C, scale, sink, pos):
    """qa [H, C], qr [H, R] of the query at position ``pos`` against cache rows [n, C + R]: float64, every key j <= pos."""
    k = rows[:pos + 1].double()
    s = (qa.double() @ k[:, :C].T + qr.double() @ k[:, C:].T) * scale          # [H, keys]
    mx = torch.maximum(s.max(-1, keepdim=True).values, sink.double()[:, None])
    e = torch.exp(s - mx)
    p = e / (e.sum(-1, keepdim=True) + torch.exp(sink.double()[:, None] - mx))
    return p @ k[:, :C]                                                          # [H, C]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, C, R, page", [(3, 40, 8, 16), (20, 16, 4, 8), (4, 136, 8, 32), (9, 64, 32, 16), (70, 24, 8, 16), (3, 40, 16, 16),
                                           (2, 264, 24, 16), (2, 512, 64, 16)])
def test_latent_attention_sees_exactly_the_keys_up_to_its_own(H, C, R, page, dtype):
    """One key stands out (it is the query's own direction, scaled), at places where a fault would show: the first token,
    a far key, the last row of a page and the first of the next, the query's own key, and the key just after the query
    (which must not be seen) with later keys of the same step already in the cache."""
    ops = _ops()
    L, q_len = 700, 40                       # a portion of 40 queries at the end of 700 keys, and single-token requests
    start = L - q_len
    gen = g(H + C)
    rows = (torch.randn(L, C + R, generator=gen) * 0.5).to(dtype)
    n_pages = (L + page - 1) // page
    perm = torch.randperm(n_pages + 5, generator=gen)[:n_pages]                  # pages in any order
    pool = torch.full(((n_pages + 5) * page, C + R), float("nan"), dtype=dtype)
    for j in range(L):
        pool[int(perm[j // page]) * page + j % page] = rows[j]
    sink = torch.randn(H, generator=gen) + 5.0
    special = [0, 3, page - 1, page, 5 * page - 1, 5 * page, 311, start - 1, start, start + 7, start + 8, L - 1]
    qa = (torch.randn(q_len, H, C, generator=gen) * 0.3)
    qr = (torch.randn(q_len, H, R, generator=gen) * 0.3)
    for i in range(q_len):                  # query i points at one of the special keys, strongly
        j = special[i % len(special)]
        qa[i, i % H] += 6.0 * rows[j, :C].float() / rows[j, :C].float().norm()
    # a query whose standout key is the one right after it: invisible
    qa[7, 1] += 6.0 * rows[start + 8, :C].float() / rows[start + 8, :C].float().norm()
    qa, qr = qa.to(dtype), qr.to(dtype)
    scale = 0.9
    # batch: two single-token requests (at positions 311 and L-1 of the same cache), then the portion
    lens, ctx = [1, 1, q_len], [312, L, L]
    meta = _meta(lens, ctx)
    T = sum(lens)
    q_abs = torch.zeros(T, H, C, dtype=dtype)
    q_rot = torch.zeros(T, H, R, dtype=dtype)
    q_abs[0], q_rot[0] = qa[3], qr[3]
    q_abs[1], q_rot[1] = qa[5], qr[5]
    q_abs[2:], q_rot[2:] = qa, qr
    bt = perm.to(torch.int32)[None].repeat(3, 1).contiguous().to(DEV)
    gate = torch.rand(T, H, generator=gen)
    out = torch.empty(H, T, C, dtype=dtype, device=DEV)
    ops.latent_attention(q_abs.transpose(0, 1).contiguous().to(DEV), q_rot.to(DEV), pool.to(DEV), page, bt, meta, sink.to(DEV),
                         gate.to(DEV), out, scale)
    got = out.cpu().float().transpose(0, 1)                                       # [T, H, C]
    positions = [311, L - 1] + list(range(start, L))
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for t, p in enumerate(positions):
        ref = _plain_rows_attention(q_abs[t], q_rot[t], rows, C, scale, sink, p) * gate[t].double()[:, None]
        assert torch.allclose(got[t].double(), ref, atol=tol, rtol=tol), f"token {t} at position {p}"
    if C > 64:
        return
    # the sink matters here (for the narrower latents, whose scores are small beside it): without it the weights would sum to one
    no_sink = _plain_rows_attention(q_abs[2], q_rot[2], rows, C, scale, torch.full((H,), -1e9), start)
    assert (no_sink - _plain_rows_attention(q_abs[2], q_rot[2], rows, C, scale, sink, start)).abs().max() > 1e-2


@pytest.mark.parametrize("rot_dims", [0, 4, 8])
def test_latent_prep_norms_rotates_and_writes_the_cache(rot_dims):
    ops = _ops()
    H, D, R, C, T, eps, base = 3, 16, 8, 40, 6, 1e-5, 5000.0
    N = H * (D + R) + C + R + H
    proj = torch.randn(T, N, generator=g(rot_dims))
    cw = torch.rand(C, generator=g(1)) + 0.5
    positions = torch.tensor([0, 1, 2, 1000, 77777, 5], dtype=torch.int32)
    slots = torch.tensor([4, 0, -1, 9, 2, 7], dtype=torch.int32)                  # -1: written nowhere
    pool = torch.zeros(10, C + R, device=DEV)
    qp, qr, gate = torch.empty(T, H, D, device=DEV), torch.empty(T, H, R, device=DEV), torch.empty(T, H, device=DEV)
    inv_freq = base ** (-torch.arange(0, rot_dims, 2, dtype=torch.float64) / max(rot_dims, 1))
    offs = {"q": 0, "c": H * (D + R), "g": H * (D + R) + C + R}
    ops.latent_prep(proj.to(DEV), offs, cw.to(DEV), eps, inv_freq.to(DEV), rot_dims, positions.to(DEV), slots.to(DEV), pool, qp, qr,
                    gate, H, D, R, C)
    p64 = proj.double()
    q = p64[:, :H * (D + R)].view(T, H, D + R)
    assert torch.allclose(qp.cpu().double(), q[..., :D], atol=1e-6)
    assert torch.allclose(qr.cpu().double(), plain.rotate_pairs(q[..., D:], positions, base, rot_dims), atol=2e-6)
    c = plain.unit_rms(p64[:, offs["c"]:offs["c"] + C], eps) * cw.double()
    kr = plain.rotate_pairs(p64[:, offs["c"] + C:offs["c"] + C + R], positions, base, rot_dims)
    for t in range(T):
        if slots[t] >= 0:
            assert torch.allclose(pool[slots[t]].cpu().double(), torch.cat((c[t], kr[t])), atol=3e-6)
    assert float(pool[[1, 3, 5, 6, 8]].abs().max()) == 0.0
    assert torch.allclose(gate.cpu().double(), torch.sigmoid(p64[:, offs["g"]:]), atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 7, 16, 40])
def test_per_head_products_and_rows(T, dtype):
    """Both up-projections in their layouts: q [T, H, D] against W_uk [H, D, C]; latents [H, T, C] against the transposed
    view of W_uv [H, V, C], then heads into rows [T, H * V]."""
    ops = _ops()
    H, D, C, V = 5, 24, 40, 12
    q = torch.randn(T, H, D, generator=g(T)).to(dtype).to(DEV)
    uk = torch.randn(H, D, C, generator=g(1)).to(dtype).to(DEV)
    out = torch.empty(H, T, C, dtype=dtype, device=DEV)
    ops.batched_heads_mm(q.transpose(0, 1), uk, out)
    ref = torch.einsum("thd,hdc->htc", q.double(), uk.double())
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out.double(), ref, atol=tol * 10, rtol=tol)
    lat = torch.randn(H, T, C, generator=g(2)).to(dtype).to(DEV)
    uv = torch.randn(H, V, C, generator=g(3)).to(dtype).to(DEV)
    ref = torch.einsum("htc,hvc->thv", lat.double(), uv.double()).reshape(T, H * V)
    heads = torch.empty(H, T, V, dtype=dtype, device=DEV)
    ops.batched_heads_mm(lat, uv.transpose(1, 2), heads)
    rows = torch.empty(T, H * V, dtype=dtype, device=DEV)
    ops.heads_to_rows(heads, rows)
    assert torch.allclose(rows.double(), ref, atol=tol * 10, rtol=tol)


def test_embedding_is_scaled_and_starts_every_stream():
    ops = _ops()
    table = torch.randn(11, 24, generator=g(0)).bfloat16()
    ids = torch.tensor([3, 10, 0], dtype=torch.int32, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    out = torch.empty(5, 3, 24, device=DEV)
    ops.embed(ids, table.to(DEV), out, err, scale=7.5)
    assert torch.equal(out.cpu(), (table[[3, 10, 0]].float() * 7.5)[None].repeat(5, 1, 1)) and not err.any()
