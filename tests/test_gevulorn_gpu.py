"""Gevulorn through the engine against the plain implementation: every way of cutting the work, several small models."""
import copy

import numpy as np
import pytest
import torch

import gevulorn_models as zoo
import helpers
import plain_gevulorn

pytestmark = pytest.mark.gpu
LENGTHS = {"A": (70, 45, 100, 33, 64, 129), "B": (37, 88, 50, 112, 41, 65), "C": (150, 33, 97, 64, 200, 41),
           "D": (61, 30, 99, 17, 70, 44)}
# Centred difference of a position's logits, root mean square over the vocabulary, relative to that of the logits: the
# worst position, and the mean over a request's positions.  bfloat16 rounds activations to 8 bits between the parts,
# which costs these narrow models a few per cent at some positions; a wrong key, state, window or sink costs tens.
TOL = {"float32": 3e-5, "bfloat16": 1e-1}
MEAN_TOL = {"float32": 1e-5, "bfloat16": 3e-2}
# In bfloat16 a router's close call may go the other way (the random weights here take no care to keep the chosen logits
# apart): that token then runs another expert and is off by tens of per cent, alone.  A model with routers may have a few
# such positions, in proportion to the router decisions a token meets on its way (a looped layer decides once a pass); in
# float32, and in a model whose routers take every expert, there is none.
FLIPS = {"float32": 0.0, "bfloat16": 0.015}
_plain = {}


def _requests(name):
    return helpers.random_requests(zoo.ALL[name][0]["vocab"], LENGTHS[name], seed=15 + zoo.ALL[name][1])


def _plain_logits(name, ids, folder=None):
    key = (folder or name, tuple(ids))
    if key not in _plain:
        cfg, w = plain_gevulorn.load_folder(folder or zoo.folder(name))
        _plain[key] = plain_gevulorn.forward(cfg, w, list(ids)).numpy()
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


def _routed(cfg):
    """How many times a token passes a router that has a choice to make."""
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [loop["times"] if loop["start"] <= i < loop["stop"] else 1 for i in range(len(cfg["layers"]))]
    return sum(n for n, l in zip(runs, cfg["layers"])
               if l["mlp"] and l["mlp"]["kind"] == "moe" and l["mlp"]["router"]["top"] < l["mlp"]["router"]["experts"])


def _check(name, dtype, reqs, got, tag, folder=None, cfg=None):
    cfg = cfg or zoo.ALL[name][0]
    for i, r in enumerate(reqs):
        ref, mine = _plain_logits(name, r, folder), got[f"{tag}{i}"]
        assert mine.shape == ref.shape and np.isfinite(mine).all()
        err = _error(mine, ref)
        bad = np.nonzero(err > TOL[dtype])[0]
        allowed = max(1, int(np.ceil(FLIPS[dtype] * len(r) * _routed(cfg)))) if _routed(cfg) and FLIPS[dtype] else 0
        assert bad.size <= allowed, (f"model {name} {dtype} cutting {tag!r} request {i}: first wrong token at position {bad[0]} "
                                     f"(error {err[bad[0]]:.3e}, tolerance {TOL[dtype]}); all: "
                                     + ", ".join(f"{p}: {err[p]:.2e}" for p in bad[:12]) + f"; median {np.median(err):.2e}")
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
    """The tails are longer than every window and chunk but C's widest, so their edges pass over decoded tokens."""
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
    assert rp.cache.state_slots.num_slots == 4 < len(reqs)         # ten requests went through four state slots
    _check(name, dtype, reqs, got, "m")


@pytest.mark.parametrize("graphs", [False, True])
def test_cutting_does_not_change_float32_logits_beyond_rounding(graphs):
    """The same request whole, token by token and in portions: the recurrence's state is carried in float32 and the
    attention's key tiles start at fixed positions, so the three differ by the order of sums alone."""
    name = "A"
    r = _requests(name)[2]
    whole, _ = _replay(name, "float32", helpers.trace_whole([r]), use_cuda_graphs=graphs)
    single, _ = _replay(name, "float32", helpers.trace_decode_tail([r], tail=len(r) - 1), use_cuda_graphs=graphs)
    parts, _ = _replay(name, "float32", helpers.trace_portions([r], sizes=(2, 5, 1, 16, 3)), use_cuda_graphs=graphs)
    for other in (single["d0"], parts["p0"]):
        assert _error(other, whole["w0"]).max() < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding(name, dtype):
    """Token by token far beyond every window and through many chunks, with pages given back on the way."""
    r = helpers.random_requests(zoo.ALL[name][0]["vocab"], (300,), seed=77)[0]
    got, rp = _replay(name, dtype, helpers.trace_decode_tail([r], tail=292), poison=True)
    _check(name, dtype, [r], got, "d")


def test_pages_behind_a_window_and_in_front_of_a_chunk_are_given_back():
    """Model A's window layers keep two first tokens and the last 20, its chunk layers the chunk of 24 being filled: a
    request of 200 tokens decoding must hold a few pages of those groups, not thirteen."""
    from mini_engine_b200.engine.replay import TraceReplayer
    name = "A"
    r = helpers.random_requests(zoo.ALL[name][0]["vocab"], (200,), seed=5)[0]
    rp = TraceReplayer(zoo.folder(name), "float32", 256, page_size=16)
    rp.run_step({"step": 0, "entries": [{"id": "x", "tokens": r[:150], "want": [149]}], "end": []})
    for p in range(150, 200):
        rp.run_step({"step": p, "entries": [{"id": "x", "tokens": [r[p]], "want": [0]}], "end": []})
    held = {(g.window, g.keep_first, g.chunk): sum(1 for p in t if p >= 0) for g, t in zip(rp.cache.groups, rp.live["x"].block_tables)}
    assert held[(20, 2, None)] <= 4 and rp.live["x"].block_tables[[g.keep_first for g in rp.cache.groups].index(2)][0] >= 0
    assert held[(None, 0, 24)] <= 3
    assert held[(33, 0, None)] <= 4


def _with(name, change):
    """A copy of a model's folder with its configuration and tensors changed by ``change(cfg, tensors)``."""
    cfg, seed, _ = zoo.ALL[name]
    cfg = copy.deepcopy(cfg)
    w = zoo.tensors(cfg, seed, zoo.RANKS[name])
    change(cfg, w)
    return cfg, zoo.write_folder(cfg, w)


def test_a_far_key_decides_the_logits():
    """Model B's second layer sees every key.  The weights of its query and key norms are scaled up so that a query's scores
    stand far apart and one key, often hundreds of tokens back, takes most of the weight: an engine that lost or
    misplaced far keys (a page's edge, a block table's row) would be wrong by far more than rounding."""
    def change(cfg, w):
        for t in ("l1.mix.q.norm", "l1.mix.k.norm"):
            w[t] = (w[t].float() * 2.5).to(torch.bfloat16)
    cfg, folder = _with("B", change)
    r = helpers.random_requests(cfg["vocab"], (420,), seed=31)[0]
    for steps, tag in ((helpers.trace_whole([r]), "w"), (helpers.trace_decode_tail([r], tail=40), "d"),
                       (helpers.trace_portions([r], sizes=(50, 2, 130, 7)), "p")):
        got, _ = _replay("B", "float32", steps, folder=folder, poison=True)
        _check("B", "float32", [r], got, tag, folder=folder, cfg=cfg)


def test_sharp_scores_at_the_edges_of_windows_and_chunks():
    """Model A with the attention layers' scales raised eightfold (normed queries and keys bound a score by scale x dim, so
    the scale is what sharpens the softmax): single keys carry the weight, and a key that is one token inside or outside a
    window, the kept first tokens or a chunk changes a position's logits by far more than rounding."""
    def change(cfg, w):
        for i in (1, 3, 4):
            cfg["layers"][i]["mixer"]["scale"] *= 8.0
        cfg["layers"][3]["mixer"]["softcap"] = 40.0
    cfg, folder = _with("A", change)
    reqs = helpers.random_requests(cfg["vocab"], (131, 77), seed=33)
    for steps, tag in ((helpers.trace_whole(reqs), "w"), (helpers.trace_decode_tail(reqs, tail=70), "d"),
                       (helpers.trace_portions(reqs, sizes=(19, 2, 24, 1, 20, 3, 47)), "p")):
        got, _ = _replay("A", "float32", steps, folder=folder, poison=True)
        _check("A", "float32", reqs, got, tag, folder=folder, cfg=cfg)


def test_a_large_sink_takes_the_weight():
    """Sinks of +6 in every head: most of the softmax's mass goes to the term without a value, so an engine that left the
    sink out (or scaled or capped it) would give outputs several times too large."""
    def change(cfg, w):
        for i in (1, 3, 4):
            w[f"l{i}.mix.sink"] = (w[f"l{i}.mix.sink"].float() + 6.0).to(torch.bfloat16)
    cfg, folder = _with("A", change)
    r = helpers.random_requests(cfg["vocab"], (90,), seed=35)[0]
    for steps, tag in ((helpers.trace_whole([r]), "w"), (helpers.trace_decode_tail([r], tail=30), "d")):
        got, _ = _replay("A", "float32", steps, folder=folder, poison=True)
        _check("A", "float32", [r], got, tag, folder=folder, cfg=cfg)
    plain_without = _plain_logits("A", r)                       # the unchanged model: the sinks matter
    assert _error(got["d0"], plain_without).max() > 1e-2


def test_a_slow_decay_remembers_the_first_tokens():
    """Model D's recurrence with a decay close to one (large positive bias, tau 64): the state holds the first tokens to
    the end, so a state that was lost or reset between portions or in a reused slot shows at every later position."""
    def change(cfg, w):
        cfg["layers"][2]["mixer"]["tau"] = 64.0
        w["l2.mix.a2.b"] = (w["l2.mix.a2.b"].float() + 4.0).to(torch.bfloat16)
    cfg, folder = _with("D", change)
    reqs = helpers.random_requests(cfg["vocab"], (150, 40, 90, 33, 70), seed=37)
    steps = helpers.trace_mixed(reqs, max_live=2, seed=4)
    got, _ = _replay("D", "float32", steps, folder=folder, poison=True, max_num_seqs=2)
    _check("D", "float32", reqs, got, "m", folder=folder, cfg=cfg)
    got, _ = _replay("D", "float32", helpers.trace_portions(reqs[:2], sizes=(2, 64, 3, 65, 1)), folder=folder)
    _check("D", "float32", reqs[:2], got, "p", folder=folder, cfg=cfg)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_one_size_replayed_from_a_graph(dtype):
    """Four portions of 130 tokens with one wanted place each: the shape comes again, so the engine records the step and
    replays it, at other positions each time (a rotation or a mask taken from the recording's positions would show)."""
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
    cfg, w = plain_gevulorn.load_folder(zoo.folder(name))
    ids = list(prompt)
    for _ in range(n):
        logits = plain_gevulorn.forward(cfg, w, ids)[-1]
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
