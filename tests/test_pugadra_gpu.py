"""Pugadra through the engine against the plain implementation: every way of cutting the work, several small models."""
import numpy as np
import pytest
import torch

import helpers
import plain_pugadra
import pugadra_models as zoo

pytestmark = pytest.mark.gpu
LENGTHS = {"A": (70, 45, 100, 33, 64, 129), "B": (37, 88, 50, 112, 41, 65), "C": (150, 33, 97, 64, 200, 41),
           "D": (61, 30, 99, 17, 70, 44)}
# Centred difference of a position's logits, root mean square over the vocabulary, relative to that of the logits: the
# worst position, and the mean over a request's positions.  bfloat16 rounds activations to 8 bits between the parts,
# which costs these narrow models a few per cent at some positions; a wrong key, state or sink costs tens of per cent.
TOL = {"float32": 2e-5, "bfloat16": 1e-1}
MEAN_TOL = {"float32": 1e-5, "bfloat16": 3e-2}
# In bfloat16 a router's close call may go the other way (the random weights here take no care to keep the chosen logits
# apart): that token then runs another expert and is off by tens of per cent, alone.  A model with routers may have a few
# such positions; in float32, and in a model whose routers take every expert, there is none.
FLIPS = {"float32": 0.0, "bfloat16": 0.03}
_plain = {}


def _requests(name):
    return helpers.random_requests(zoo.ALL[name][0]["vocab"], LENGTHS[name], seed=5 + zoo.ALL[name][1])


def _plain_logits(name, ids):
    key = (name, tuple(ids))
    if key not in _plain:
        cfg, w = plain_pugadra.load_folder(zoo.folder(name))
        _plain[key] = plain_pugadra.forward(cfg, w, list(ids)).numpy()
    return _plain[key]


def _error(mine, ref):
    d = mine - ref
    d = d - d.mean(axis=1, keepdims=True)
    r = ref - ref.mean(axis=1, keepdims=True)
    return np.sqrt((d ** 2).mean(axis=1)) / np.sqrt((r ** 2).mean())


def _replay(name, dtype, steps, max_tokens=None, folder=None, **kw):
    from mini_engine_b200.engine.replay import TraceReplayer
    rp = TraceReplayer(folder or zoo.folder(name), dtype, max_tokens or helpers.max_live_tokens(steps), page_size=zoo.ALL[name][2], **kw)
    outs = [rp.run_step(st) for st in steps]
    assert not rp.live
    rp.cache.check([])
    assert rp.cache.num_free_pages == [p.num_pages for p in rp.cache.pools]
    assert rp.cache.state_slots.num_free == rp.cache.state_slots.num_slots
    return helpers.collect(steps, outs), rp


def _check(name, dtype, reqs, got, tag):
    for i, r in enumerate(reqs):
        ref, mine = _plain_logits(name, r), got[f"{tag}{i}"]
        assert mine.shape == ref.shape and np.isfinite(mine).all()
        err = _error(mine, ref)
        bad = np.nonzero(err > TOL[dtype])[0]
        routed = any(l["mlp"] and l["mlp"]["kind"] == "moe" and l["mlp"]["router"]["top"] < l["mlp"]["router"]["experts"]
                     for l in zoo.ALL[name][0]["layers"])
        assert bad.size <= (max(1, int(FLIPS[dtype] * len(r))) if routed and FLIPS[dtype] else 0), (f"model {name} {dtype} cutting {tag!r} request {i}: first wrong token at position {bad[0]} "
                               f"(error {err[bad[0]]:.3e}, tolerance {TOL[dtype]})")
        assert np.median(err) < MEAN_TOL[dtype] and err.mean() < 3 * MEAN_TOL[dtype], f"model {name} {dtype} cutting {tag!r} request {i}: mean error {err.mean():.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_each_request_alone_and_whole(name, dtype):
    reqs = _requests(name)
    got, _ = _replay(name, dtype, helpers.trace_whole(reqs), poison=True)
    _check(name, dtype, reqs, got, "w")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_prompt_then_token_by_token(name, dtype):
    """The tails are longer than every window but C's widest, so windows pass over decoded tokens."""
    reqs = _requests(name)
    got, _ = _replay(name, dtype, helpers.trace_decode_tail(reqs, tail=60), poison=True)
    _check(name, dtype, reqs, got, "d")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_of_changing_size(name, dtype):
    reqs = _requests(name)
    got, _ = _replay(name, dtype, helpers.trace_portions(reqs), poison=True)
    _check(name, dtype, reqs, got, "p")
    got, _ = _replay(name, dtype, helpers.trace_portions(reqs, sizes=(2, 2, 3, 1, 2, 17, 2, 31)), poison=True)
    _check(name, dtype, reqs, got, "p")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_batches_with_pages_and_slots_used_again(name, dtype):
    reqs = _requests(name) + _requests(name)[:4]
    steps = helpers.trace_mixed(reqs, max_live=4, seed=3)
    assert max(len(st["entries"]) for st in steps) >= 3
    assert any(len(e["tokens"]) == 1 for st in steps for e in st["entries"] if len(st["entries"]) > 1)
    need = helpers.max_live_tokens(steps)
    assert need < sum((len(r) + 63) // 64 * 64 for r in reqs)
    got, rp = _replay(name, dtype, steps, max_tokens=need, poison=True)
    if name != "D":                                                # (D has no convolution, so no state)
        assert rp.cache.state_slots.num_slots == 4 < len(reqs)     # ten requests went through four state slots
    _check(name, dtype, reqs, got, "m")


@pytest.mark.parametrize("graphs", [False, True])
def test_cutting_does_not_change_float32_logits_beyond_rounding(graphs):
    """The same request whole, token by token and in portions: the convolution's state is carried exactly and the
    attention's key tiles start at fixed positions, so the three differ by the products' rounding alone."""
    name = "A"
    r = _requests(name)[2]
    whole, _ = _replay(name, "float32", helpers.trace_whole([r]), use_cuda_graphs=graphs)
    single, _ = _replay(name, "float32", helpers.trace_decode_tail([r], tail=len(r) - 1), use_cuda_graphs=graphs)
    parts, _ = _replay(name, "float32", helpers.trace_portions([r], sizes=(2, 5, 1, 16, 3)), use_cuda_graphs=graphs)
    for other in (single["d0"], parts["p0"]):
        assert _error(other, whole["w0"]).max() < 5e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """Token by token far beyond every window, with pages of the window groups given back on the way."""
    name = "A"
    r = helpers.random_requests(zoo.ALL[name][0]["vocab"], (300,), seed=77)[0]
    got, rp = _replay(name, dtype, helpers.trace_decode_tail([r], tail=292), poison=True)
    _check(name, dtype, [r], got, "d")


def test_a_far_key_decides_the_logits():
    """Model A's third layer sees every key.  Its query and key projections are scaled up so that a query's scores stand
    far apart and one key, often hundreds of tokens back, takes most of the weight: an engine that lost or misplaced far
    keys (a page's edge, a block table's row) would be wrong by far more than rounding."""
    name = "A"
    cfg, seed, _ = zoo.ALL[name]
    w = zoo.tensors(cfg, seed)
    for t in ("l2.mix.q", "l2.mix.k"):
        w[t] = (w[t].float() * 3.0).to(torch.bfloat16)
    folder = zoo.write_folder(cfg, w)
    r = helpers.random_requests(cfg["vocab"], (420,), seed=31)[0]
    c, ww = plain_pugadra.load_folder(folder)
    ref = plain_pugadra.forward(c, ww, r).numpy()
    for steps, tag in ((helpers.trace_whole([r]), "w"), (helpers.trace_decode_tail([r], tail=40), "d"),
                       (helpers.trace_portions([r], sizes=(50, 2, 130, 7)), "p")):
        got, _ = _replay(name, "float32", steps, folder=folder, poison=True)
        assert _error(got[f"{tag}0"], ref).max() < 5e-5, tag


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_one_size_replayed_from_a_graph(dtype):
    """Four portions of 130 tokens with one wanted place each: the shape comes again, so the engine records the step and
    replays it, at other positions each time (a rotation taken from the recording's positions would show at once)."""
    name = "C"
    r = helpers.random_requests(zoo.ALL[name][0]["vocab"], (520,), seed=41)[0]
    steps = [{"step": k, "entries": [{"id": "g0", "tokens": r[130 * k:130 * (k + 1)], "want": [129]}], "end": ["g0"] if k == 3 else []}
             for k in range(4)]
    got, rp = _replay(name, dtype, steps)
    assert rp.runner._prefill_graphs, "the step was never replayed from a graph"
    ref = _plain_logits(name, r)[[129, 259, 389, 519]]
    err = _error(got["g0"], ref)
    assert err.max() < (TOL[dtype] if dtype == "float32" else 0.15), err


def _plain_greedy(name, prompt, n):
    cfg, w = plain_pugadra.load_folder(zoo.folder(name))
    ids = list(prompt)
    for _ in range(n):
        logits = plain_pugadra.forward(cfg, w, ids)[-1]
        top = torch.topk(logits, 2).values
        if float(top[0] - top[1]) < 1e-3:                # a tie within rounding: the comparison stops here
            break
        ids.append(int(torch.argmax(logits)))
    return ids[len(prompt):]


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_engine(name):
    """``LLM.generate`` with the scheduler cutting prompts into portions and batching them with decoding requests."""
    from mini_engine_b200.llm import LLM
    from mini_engine_b200.sampling.params import SamplingParams
    vocab = zoo.ALL[name][0]["vocab"]
    prompts = helpers.random_requests(vocab, (21, 5, 40, 9, 33), seed=9)
    llm = LLM(zoo.folder(name), dtype="float32", kvcache_block_size=zoo.ALL[name][2], num_kvcache_blocks=24, max_num_seqs=3,
              max_num_batched_tokens=16, max_model_len=128)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        want = _plain_greedy(name, p, 12)
        assert len(want) >= 4
        assert o["token_ids"][:len(want)] == want
