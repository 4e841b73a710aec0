"""Each mechanism of Pugadra alone: the kernel behind it against the plain function, on inputs made so that a fault shows."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_pugadra as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _ops():
    from mini_engine_b200 import ops
    ops.require_extension()
    return ops


def _meta(lens, contexts):
    """Step metadata as the kernels read it: requests that bring one token come first."""
    D = sum(1 for n in lens if n == 1)
    assert all(n == 1 for n in lens[:D])
    cu = np.concatenate(([0], np.cumsum(lens))).astype(np.int32)
    token_req = torch.tensor(np.repeat(np.arange(len(lens)), lens), dtype=torch.int32, device=DEV)
    positions = torch.tensor(np.concatenate([np.arange(c - n, c) for n, c in zip(lens, contexts)]), dtype=torch.int32, device=DEV)
    lists = {}
    for tq in (8, 16, 32, 64, 128):
        tiles = [(b, q0) for b in range(D, len(lens)) for q0 in range(0, lens[b], tq)]
        lists[tq] = (torch.tensor(tiles or [(0, 0)], dtype=torch.int32, device=DEV), len(tiles))
    meta = SimpleNamespace(cu_seqlens=torch.tensor(cu, device=DEV), context_lens=torch.tensor(contexts, dtype=torch.int32, device=DEV),
                           num_reqs=len(lens), num_tokens=int(cu[-1]), num_decodes=D, tile_lists=lists, num_tiles=len(lists[16][0]),
                           max_context_len=max(contexts), error_flag=None,
                           workspace=lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=DEV))
    return meta, token_req, positions


def g(seed):
    return torch.Generator().manual_seed(seed)


# ---- the norm on both sides of a sub-layer -------------------------------------------------------------------
@pytest.mark.parametrize("W", [40, 200, 1030, 4100])
def test_scaled_normed_update_and_the_next_norm(W):
    ops = _ops()
    T, eps, mult = 6, 1e-5, 0.3
    x = torch.randn(T, W, generator=g(W)) * 2 + 0.3
    y = torch.randn(T, W, generator=g(1)) * 5
    wb, wa = torch.randn(W, generator=g(2)) * 0.3, torch.randn(W, generator=g(3)) * 0.3
    new = x.double() + mult * plain.norm_around_zero(y.double(), wb.double(), eps)
    ref = plain.norm_around_zero(new, wa.double(), eps)
    xd, out = x.to(DEV), torch.empty(T, W, device=DEV)
    ops.sandwich_norm(xd, y.to(DEV), (1 + wb).to(DEV), mult, (1 + wa).to(DEV), eps, out)
    assert torch.allclose(xd.cpu().double(), new, atol=1e-5) and torch.allclose(out.cpu().double(), ref, atol=2e-5)
    # the stream itself, rounded, for a reader that takes no norm; a bfloat16 update
    xd2, out2 = x.to(DEV), torch.empty(T, W, device=DEV, dtype=torch.bfloat16)
    ops.sandwich_norm(xd2, y.to(DEV).bfloat16(), (1 + wb).to(DEV), mult, None, eps, out2, norm_out=False)
    new2 = x.double() + mult * plain.norm_around_zero(y.bfloat16().double(), wb.double(), eps)
    assert torch.allclose(xd2.cpu().double(), new2, atol=1e-5) and torch.equal(out2.cpu(), xd2.cpu().bfloat16())
    # two rows only, nothing written; and no update at all
    xd3, rows, out3 = x.to(DEV), torch.tensor([4, 1], dtype=torch.int32, device=DEV), torch.empty(2, W, device=DEV)
    ops.sandwich_norm(xd3, y.to(DEV), (1 + wb).to(DEV), mult, (1 + wa).to(DEV), eps, out3, rows=rows)
    assert torch.equal(xd3.cpu(), x) and torch.allclose(out3.cpu().double(), ref[[4, 1]], atol=2e-5)
    ops.sandwich_norm(xd3, None, None, mult, (1 + wa).to(DEV), eps, out)
    assert torch.allclose(out.cpu().double(), plain.norm_around_zero(x.double(), wa.double(), eps), atol=2e-5)


def test_the_update_is_normalised_before_it_is_added():
    """An update a thousand times larger must change the stream by the same amount."""
    ops = _ops()
    W = 64
    x, y, w = torch.randn(3, W, generator=g(0)), torch.randn(3, W, generator=g(1)), torch.ones(W)
    a, b = x.to(DEV), x.to(DEV)
    ops.sandwich_norm(a, y.to(DEV), w.to(DEV), 0.5, None, 1e-9, None)
    ops.sandwich_norm(b, (y * 1000).to(DEV), w.to(DEV), 0.5, None, 1e-9, None)
    assert torch.allclose(a, b, atol=1e-4) and not torch.allclose(a.cpu(), x, atol=0.1)


# ---- bias, convolution with state, rotation, cache write -----------------------------------------------------
@pytest.mark.parametrize("taps, H, G, D, V, rot, own_kv", [(3, 4, 2, 16, 24, 8, True), (1, 3, 1, 10, 9, 6, True), (4, 6, 3, 6, 5, 0, True),
                                                          (2, 5, 5, 8, 8, 8, False), (0, 2, 1, 12, 7, 12, True), (6, 2, 2, 8, 6, 4, True)])
@pytest.mark.parametrize("table", [False, True])
def test_projections_through_convolution_and_rotation_in_portions_with_slots_used_again(taps, H, G, D, V, rot, own_kv, table):
    """``table``: the cosines and sines come from the step's table instead of being formed by every thread."""
    ops = _ops()
    ps, pages, slots, base = 8, 24, 3, 700.0
    C = H * D + (G * (D + V) if own_kv else 0)
    extra = 5                                                  # columns behind the channels (the gate's), left alone
    lens_total = (23, 9, 31)
    proj = [torch.randn(n, C + extra, generator=g(10 + n)) for n in lens_total]
    bias = torch.randn(C, generator=g(1)) * 0.5
    wt = torch.randn(C, max(taps, 1), generator=g(2)) * 0.6
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64)
    ref_q, ref_kv = [], []
    for p in proj:
        u = p[:, :C].double() + bias.double()
        y = plain.causal_conv(u, wt.double()) if taps else u
        pos = torch.arange(p.shape[0])
        ref_q.append(plain.rotate_pairs(y[:, :H * D].reshape(-1, H, D), pos, base, rot))
        if own_kv:
            k = plain.rotate_pairs(y[:, H * D:H * D + G * D].reshape(-1, G, D), pos, base, rot)
            ref_kv.append((k, y[:, H * D + G * D:].reshape(-1, G, V)))
    state = torch.full((slots, max(taps - 1, 1), C), float("nan"), device=DEV)[:, :max(taps - 1, 0)].contiguous()
    HD = max(D, V) + 3                                        # cache rows may be longer than a key or a value
    pool = torch.full((pages, 2, G, ps, HD), float("nan"), device=DEV)
    perm = torch.randperm(pages, generator=g(3)).tolist()
    tables = [perm[0:3], perm[3:5], perm[5:9]]
    slot_of = [2, 0, 2]                                     # request 2 takes request 0's slot once that has ended
    got = [[] for _ in proj]
    plan = [[(1, 1), (0, 5)], [(0, 1), (1, 2)], [(1, 1), (0, 2)], [(0, 1), (1, 5)], [(0, 14)], [(2, 2)], [(2, 1)], [(2, 1)], [(2, 27)]]
    pos = [0, 0, 0]
    for step in plan:
        lens = [n for _, n in step]
        h = torch.cat([proj[r][pos[r]:pos[r] + n] for r, n in step]).to(DEV)
        meta, token_req, positions = _meta(lens, [pos[r] + n for r, n in step])
        sm = torch.tensor([tables[r][(pos[r] + i) // ps] * ps + (pos[r] + i) % ps for r, n in step for i in range(n)],
                          dtype=torch.int32, device=DEV)
        ctx = SimpleNamespace(attn_meta=meta, token_req=token_req, positions=positions,
                              state_slots=torch.tensor([slot_of[r] for r, _ in step], dtype=torch.int32, device=DEV))
        q = torch.empty(h.shape[0], H * D, device=DEV)
        angles = None
        if table and rot:
            angles = torch.empty(h.shape[0], rot // 2, 2, device=DEV)
            ops.rope_table(positions, inv_freq.to(DEV), angles)
        ops.conv_rope_kv(h, bias.to(DEV), wt.to(DEV) if taps else None, state if taps > 1 else None, inv_freq.to(DEV), rot, ctx,
                         sm if own_kv else None, q, pool if own_kv else None, ps, H, G, D, V, own_kv, angles=angles)
        o = 0
        for r, n in step:
            got[r].append(q[o:o + n].cpu())
            o += n
            pos[r] += n
    for r in range(3):
        n = pos[r]
        assert torch.allclose(torch.cat(got[r]).double().view(n, H, D), ref_q[r][:n], atol=2e-5), f"queries of request {r}"
        if own_kv and r != 0:                               # (request 0 ended; nothing reused its pages here)
            rows = torch.stack([pool[tables[r][j // ps], :, :, j % ps] for j in range(n)]).cpu().double()     # [n, 2, G, HD]
            assert torch.allclose(rows[:, 0, :, :D], ref_kv[r][0][:n], atol=2e-5), f"cached keys of request {r}"
            assert torch.allclose(rows[:, 1, :, :V], ref_kv[r][1][:n], atol=2e-5), f"cached values of request {r}"
            assert torch.isnan(rows[:, 0, :, D:]).all() and torch.isnan(rows[:, 1, :, V:]).all()


# ---- attention with a window, a sink and a gate ---------------------------------------------------------------
def _paged(keys, values, ps, dtype, seed):
    """The keys and values of several requests in pages handed out in a shuffled order: [pages, 2, kv heads, page, row]."""
    need = [(k.shape[0] + ps - 1) // ps for k in keys]
    pages = sum(need) + 3
    G, D, V = keys[0].shape[1], keys[0].shape[2], values[0].shape[2]
    pool = torch.full((pages, 2, G, ps, max(D, V)), float("nan"), dtype=dtype, device=DEV)
    perm = torch.randperm(pages, generator=g(seed)).tolist()
    bt = torch.full((len(keys), max(need)), -1, dtype=torch.int32)
    for b, (k, v) in enumerate(zip(keys, values)):
        for i in range(need[b]):
            page = perm.pop()
            bt[b, i] = page
            n = k[i * ps:(i + 1) * ps].shape[0]
            pool[page, 0, :, :n, :D] = k[i * ps:(i + 1) * ps].transpose(0, 1).to(dtype).to(DEV)
            pool[page, 1, :, :n, :V] = v[i * ps:(i + 1) * ps].transpose(0, 1).to(dtype).to(DEV)
    return pool, bt.to(DEV)


def _attention_case(ops, dtype, H, G, D, V, window, sink, ps, lens, contexts, seed, boost=None, gate=True):
    """Runs the kernel on requests whose last ``lens`` tokens are this step's queries; returns (got, reference) per request."""
    dt = DT[dtype]
    scale = 0.37
    qs = [torch.randn(c, H, D, generator=g(seed + i)) for i, c in enumerate(contexts)]
    ks = [torch.randn(c, G, D, generator=g(seed + 10 + i)) for i, c in enumerate(contexts)]
    vs = [torch.randn(c, G, V, generator=g(seed + 20 + i)) for i, c in enumerate(contexts)]
    gs = [torch.randn(c, H * V, generator=g(seed + 30 + i)) * 2 for i, c in enumerate(contexts)]
    if boost:
        boost(qs, ks)
    qs, ks, vs = ([t.to(dt).float() for t in ts] for ts in (qs, ks, vs))       # what the kernel is given, exactly
    pool, bt = _paged(ks, vs, ps, dt, seed)
    meta, _, _ = _meta(list(lens), list(contexts))
    meta.error_flag = torch.zeros(4, dtype=torch.int32, device=DEV)
    q = torch.cat([qq[c - n:].reshape(n, H * D) for qq, n, c in zip(qs, lens, contexts)]).to(dt).to(DEV)
    gate_rows = torch.cat([gg[c - n:] for gg, n, c in zip(gs, lens, contexts)]).to(DEV) if gate else None
    out = torch.empty(q.shape[0], H * V, dtype=dt, device=DEV)
    ops.sink_attention(q, gate_rows, out, pool, ps, bt, meta, H, G, D, V, scale, window, sink)
    assert not meta.error_flag.any()
    res, o = [], 0
    for qq, kk, vv, gg, n, c in zip(qs, ks, vs, gs, lens, contexts):
        ref = _plain_attention(qq.double(), kk.double(), vv.double(), scale, window, sink)[c - n:].reshape(n, H * V)
        if gate:
            ref = ref * torch.sigmoid(gg[c - n:].double())
        res.append((out[o:o + n].float().cpu().double(), ref))
        o += n
    return res


def _plain_attention(q, k, v, scale, window, sink):
    if sink:
        return plain.windowed_sink_attention(q, k, v, scale, window)
    # without the sink: an ordinary softmax over the same keys (the kernel's other branch)
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for h in range(H):
            gq = h // (H // k.shape[1])
            p = torch.softmax((k[lo:i + 1, gq] @ q[i, h]) * scale, 0)
            out[i, h] = (p[:, None] * v[lo:i + 1, gq]).sum(0)
    return out


ATOL = {"float32": 2e-5, "bfloat16": 2e-2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, D, V, window, ps", [(4, 2, 16, 24, 40, 16), (3, 1, 10, 9, 33, 8), (10, 2, 40, 40, 72, 16),
                                                    (8, 2, 64, 64, 128, 16), (4, 4, 32, 64, None, 32), (2, 2, 8, 8, 1, 16),
                                                    (8, 1, 128, 128, 200, 64), (5, 5, 6, 5, 7, 8)])
def test_attention_in_prompts_and_single_tokens(dtype, H, G, D, V, window, ps):
    """Single tokens (first in the batch), a prompt from position 0, portions that start in the middle of a page and of a
    window, a portion of two tokens."""
    ops = _ops()
    lens, contexts = (1, 1, 1, 70, 45, 2, 150), (1, 97, 300, 70, 211, 130, 150)
    for (got, ref) in _attention_case(ops, dtype, H, G, D, V, window, True, ps, lens, contexts, seed=H * D):
        assert torch.allclose(got, ref, atol=ATOL[dtype], rtol=1e-2 if dtype == "bfloat16" else 1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_without_sink_and_without_gate(dtype):
    ops = _ops()
    for (got, ref) in _attention_case(ops, dtype, 4, 2, 16, 16, 20, False, 16, (1, 33, 64), (50, 80, 64), seed=3, gate=False):
        assert torch.allclose(got, ref, atol=ATOL[dtype], rtol=1e-2 if dtype == "bfloat16" else 1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window, ps, D", [(40, 16, 16), (33, 8, 10), (72, 16, 40), (128, 16, 64), (64, 64, 64)])
@pytest.mark.parametrize("delta", [0, 1])
def test_a_key_at_the_windows_edge(dtype, window, ps, D, delta):
    """One key gets a score far above the others: the last one inside the window (delta 0: nearly all the weight must go
    to its value) or the first one outside (delta 1: it must not be seen at all), for a single token and inside a prompt."""
    ops = _ops()
    H, G, V = 2, 1, D
    lens, contexts = (1, 60), (window + 140, window + 140)

    def boost(qs, ks):
        for qq, kk in zip(qs, ks):
            for p in (qq.shape[0] - 1, qq.shape[0] - 7):        # the decoded token; a token inside the prompt's portion
                j = p - window + 1 - delta
                kk[j] = qq[p, 0:1] * (30.0 / 0.37) / (qq[p, 0] ** 2).sum()
    res = _attention_case(ops, dtype, H, G, D, V, window, True, ps, lens, contexts, seed=11 + window, boost=boost, gate=False)
    for (got, ref), n in zip(res, lens):
        assert torch.allclose(got, ref, atol=ATOL[dtype], rtol=1e-2 if dtype == "bfloat16" else 1e-5)


def test_the_sink_takes_its_share():
    """With every score far below zero the sink holds almost all of the weight: the output is nearly nothing."""
    ops = _ops()

    def boost(qs, ks):
        for qq, kk in zip(qs, ks):
            qq[:] = 1.0
            kk[:] = -3.0
    for sink, small in ((True, True), (False, False)):
        (got, ref), = _attention_case(ops, "float32", 2, 1, 16, 16, 24, sink, 16, (30,), (90,), seed=5, boost=boost, gate=False)
        assert torch.allclose(got, ref, atol=2e-5)
        assert (got.abs().max() < 1e-3) == small


# ---- feed-forwards -----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("limit", [None, 0.8])
def test_clamped_gated_activation(dtype, limit):
    ops = _ops()
    T, F = 9, 70
    z = (torch.randn(T, 2 * F, generator=g(0)) * 2).to(DT[dtype])
    gate, up = z[:, :F].double(), z[:, F:].double()
    if limit is not None:
        gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
        assert (z[:, :F].double() < -limit).any()              # the gate is clamped from above only
    ref = gate * torch.sigmoid(1.702 * gate) * (up + 1)
    out = torch.empty(T, F, dtype=DT[dtype], device=DEV)
    ops.clamped_glu(z.to(DEV), out, limit or 0.0, 1.702)
    assert torch.allclose(out.float().cpu().double(), ref, atol=ATOL[dtype], rtol=1e-2 if dtype == "bfloat16" else 1e-5)


@pytest.mark.parametrize("limit", [None, 0.9])
@pytest.mark.parametrize("T, W, F", [(256, 128, 192), (2048, 256, 1024), (300, 72, 200), (8, 128, 192), (5, 4096, 264), (16, 1024, 520)])
def test_clamped_gated_activation_as_the_epilogue_of_the_products(limit, T, W, F):
    """The gate|up product with the activation in its epilogue against the plain function: a long step (the one-tile and the
    persistent form of the tcgen05 product) and a step of up to 16 tokens (the decode product, and its streaming form from
    K 3,072 on)."""
    ops = _ops()
    h = torch.randn(T, W, generator=g(1)).bfloat16()
    w = {"gate": (torch.randn(F, W, generator=g(2)) * 0.2).bfloat16(), "up": (torch.randn(F, W, generator=g(3)) * 0.2).bfloat16()}
    gate, up = h.double() @ w["gate"].double().T, h.double() @ w["up"].double().T
    if limit is not None:
        gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
    ref = gate * torch.sigmoid(1.702 * gate) * (up + 1)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    out = torch.empty(T, F, dtype=torch.bfloat16, device=DEV)
    packed = torch.cat((w["gate"], w["up"])).to(DEV).contiguous()
    if T > 16:
        ops.linear_tcgen05(h.to(DEV), packed, out, "silu_mul", err, glu=(limit or 0.0, 1.702, 1.0))
    else:
        assert ops.decode_linear_takes(T, W, packed, False)
        ops.decode_linear(packed, h.to(DEV), out=out, epilogue="silu_mul", err=err, glu=(limit or 0.0, 1.702, 1.0))
    assert not err.any()
    assert torch.allclose(out.float().cpu().double(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T, E, top, W, F", [(37, 6, 2, 64, 40), (5, 5, 3, 52, 22), (130, 16, 2, 128, 64), (64, 3, 3, 40, 24),
                                             (1, 4, 1, 64, 32), (300, 11, 1, 96, 160), (700, 8, 2, 200, 320), (1100, 5, 1, 72, 200)])
def test_routed_experts_against_the_plain_loop(dtype, T, E, top, W, F):
    """Routing, grouping by expert, both products and the weighted sum, with and without a shared expert's output."""
    ops = _ops()
    dt = DT[dtype]
    w = {"router": torch.randn(E, W, generator=g(1)) * 0.5, "router.b": torch.randn(E, generator=g(2))}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = torch.randn(F, W, generator=g(10 + e)) * 0.3, torch.randn(F, W, generator=g(40 + e)) * 0.3
        w[f"e{e}.down"] = torch.randn(W, F, generator=g(70 + e)) * 0.2
    w = {k: v.to(dt).double() for k, v in w.items()}
    h = torch.randn(T, W, generator=g(3)).to(dt)
    shared = torch.randn(T, W, generator=g(4)).to(dt)
    mlp = {"router": {"experts": E, "top": top}, "expert": {"limit": 1.1}}
    ref = plain.routed_experts(h.double(), w, "", mlp) + shared.double()
    hd = h.to(DEV)
    z = (hd.float() @ w["router"].float().to(DEV).T).contiguous()
    idx, wgt = torch.empty(T, top, dtype=torch.int32, device=DEV), torch.empty(T, top, device=DEV)
    ops.moe_route(z, w["router.b"].float().to(DEV), top, idx, wgt)
    logits = z.cpu().double() + w["router.b"]
    want_idx = torch.topk(logits, top).indices
    assert torch.equal(idx.cpu().long(), want_idx)
    assert torch.allclose(wgt.cpu().double(), torch.softmax(torch.gather(logits, 1, want_idx), 1), atol=1e-6)
    counts, offsets = torch.empty(E, dtype=torch.int32, device=DEV), torch.empty(E + 1, dtype=torch.int32, device=DEV)
    order, place = torch.empty(T * top, dtype=torch.int32, device=DEV), torch.empty(T * top, dtype=torch.int32, device=DEV)
    ops.moe_sort(idx, E, counts, offsets, order, place)
    flat = idx.cpu().flatten()
    assert offsets.cpu().tolist() == [0] + torch.cumsum(torch.bincount(flat, minlength=E), 0).tolist()
    assert sorted(order.cpu().tolist()) == list(range(T * top)) and torch.equal(order[place.long()].cpu(), torch.arange(T * top, dtype=torch.int32))
    by_expert = flat[order.cpu().long()]
    assert torch.equal(by_expert, by_expert.sort().values)
    # routing and grouping in one call (one kernel for few tokens) gives the same
    both = [torch.empty_like(t) for t in (idx, wgt, counts, offsets, order, place)]
    ops.moe_route_sort(z, w["router.b"].float().to(DEV), top, *both)
    assert all(torch.equal(a, b) for a, b in zip((idx, wgt, offsets, order, place), (both[0], both[1], both[3], both[4], both[5])))
    gate_up = torch.stack([torch.cat((w[f"e{e}.gate"], w[f"e{e}.up"])) for e in range(E)]).to(dt).to(DEV).contiguous()
    down = torch.stack([w[f"e{e}.down"] for e in range(E)]).to(dt).to(DEV).contiguous()
    act, rows = torch.empty(T * top, F, dtype=dt, device=DEV), torch.empty(T * top, W, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    work = lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=DEV)
    ops.moe_gemm(hd, order, top, gate_up, offsets, act, glu=(1.1, 1.702), workspace=work, err=err)      # 512 pairs and more: tcgen05
    ops.moe_gemm(act, None, top, down, offsets, rows, workspace=work, err=err)
    assert not err.any()
    out = torch.empty(T, W, dtype=dt, device=DEV)
    ops.moe_combine(rows, place, wgt, shared.to(DEV), out)
    assert torch.allclose(out.float().cpu().double(), ref, atol=ATOL[dtype] * 3, rtol=2e-2 if dtype == "bfloat16" else 1e-5)
    ops.moe_combine(rows, place, wgt, None, out)
    assert torch.allclose(out.float().cpu().double(), ref - shared.double(), atol=ATOL[dtype] * 3, rtol=2e-2 if dtype == "bfloat16" else 1e-5)


# ---- the token's own input ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_slice_of_the_second_embedding(dtype):
    ops = _ops()
    T, dim, layers, vocab, layer = 11, 6, 4, 50, 2
    z = torch.randn(T, dim, generator=g(0)) * 2
    table = torch.randn(vocab, dim * layers, generator=g(1)).to(DT[dtype])
    ids = torch.randint(0, vocab, (T,), generator=g(2), dtype=torch.int32)
    ref = plain.gelu_tanh(z.double()) * table.double()[ids.long()][:, layer * dim:(layer + 1) * dim]
    out = torch.empty(T, dim, dtype=DT[dtype], device=DEV)
    ops.token_side_gate(z.to(DEV), ids.to(DEV), None, table.to(DEV), layer * dim, out)
    assert torch.allclose(out.float().cpu().double(), ref, atol=ATOL[dtype], rtol=1e-2 if dtype == "bfloat16" else 1e-5)
