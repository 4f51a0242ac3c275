"""Galupel through the engine against the plain implementation: every way of cutting the work, several small models."""
import copy

import numpy as np
import pytest
import torch

import galupel_models as zoo
import helpers
import plain_galupel

pytestmark = pytest.mark.gpu
LENGTHS = {"A": (70, 45, 100, 33, 64, 129), "B": (37, 88, 50, 112, 41, 65), "C": (150, 33, 97, 64, 200, 41),
           "D": (210, 47, 130, 64, 300, 95)}
# Centred difference of a position's logits, root mean square over the vocabulary, relative to that of the logits: the
# worst position, and the mean over a request's positions.  bfloat16 rounds activations to 8 bits between the parts,
# which costs these narrow models a few per cent at some positions; a wrong key, block, window or expert costs tens.
TOL = {"float32": 3e-5, "bfloat16": 1e-1}
MEAN_TOL = {"float32": 1e-5, "bfloat16": 3e-2}
# In bfloat16 a router's close call may go the other way (the random weights here take no care to keep the choice scores
# apart, and a router decides twice: which groups, then which experts): that token then runs other experts and is off by
# tens of per cent, alone.  A model with routers may have a few such positions, in proportion to the router decisions a
# token meets on its way; in float32, and in a model whose routers take every expert, there is none.
FLIPS = {"float32": 0.0, "bfloat16": 0.04}
_plain = {}


def _requests(name):
    return helpers.random_requests(zoo.ALL[name][0]["vocab"], LENGTHS[name], seed=25 + zoo.ALL[name][1])


def _plain_logits(name, ids, folder=None):
    key = (folder or name, tuple(ids))
    if key not in _plain:
        cfg, w = plain_galupel.load_folder(folder or zoo.folder(name))
        _plain[key] = plain_galupel.forward(cfg, w, list(ids)).numpy()
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
    return helpers.collect(steps, outs), rp


def _routed(cfg):
    """How many routers with a choice to make a token passes."""
    return sum(1 for l in cfg["layers"] if l["mlp"] and l["mlp"]["router"]["top"] < l["mlp"]["router"]["experts"])


def _check(name, dtype, reqs, got, tag, folder=None, cfg=None, tol=None):
    """``tol``: for models whose scores were sharpened (a float32 score of 40 carries a rounding of 4e-6 into the exponent)."""
    cfg = cfg or zoo.ALL[name][0]
    tol = tol or TOL[dtype]
    for i, r in enumerate(reqs):
        ref, mine = _plain_logits(name, r, folder), got[f"{tag}{i}"]
        assert mine.shape == ref.shape and np.isfinite(mine).all()
        err = _error(mine, ref)
        bad = np.nonzero(err > tol)[0]
        allowed = max(1, int(np.ceil(FLIPS[dtype] * len(r) * _routed(cfg)))) if _routed(cfg) and FLIPS[dtype] else 0
        assert bad.size <= allowed, (f"model {name} {dtype} cutting {tag!r} request {i}: first wrong token at position {bad[0]} "
                                     f"(error {err[bad[0]]:.3e}, tolerance {tol}); all: "
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
    """The tails are longer than every window and block but C's widest, so their edges pass over decoded tokens."""
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
def test_mixed_batches_with_pages_used_again(name, dtype):
    reqs = _requests(name) + _requests(name)[:4]
    steps = helpers.trace_mixed(reqs, max_live=4, seed=3)
    assert max(len(st["entries"]) for st in steps) >= 3
    assert any(len(e["tokens"]) == 1 for st in steps for e in st["entries"] if len(st["entries"]) > 1)
    need = helpers.max_live_tokens(steps)
    assert need < sum((len(r) + 63) // 64 * 64 for r in reqs)
    got, rp = _replay(name, dtype, steps, max_tokens=need, poison=True)
    _check(name, dtype, reqs, got, "m")


@pytest.mark.parametrize("graphs", [False, True])
def test_cutting_does_not_change_float32_logits_beyond_rounding(graphs):
    """The same request whole, token by token and in portions: key tiles start at fixed positions and a block's means are
    formed once, from the cache, so the three differ by the order of sums alone."""
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
    """Token by token far beyond every window and through dozens of blocks, with pages given back on the way."""
    r = helpers.random_requests(zoo.ALL[name][0]["vocab"], (300,), seed=77)[0]
    got, rp = _replay(name, dtype, helpers.trace_decode_tail([r], tail=292), poison=True)
    _check(name, dtype, [r], got, "d")


def test_pages_behind_a_window_are_given_back_and_blocks_are_kept():
    """Model A's first layer lends its keys to windows of 20, 7 and 11 tokens and blocks of 5, 3 and 16: a request of 200 tokens
    decoding holds the few token pages that the widest of them needs, and all of the blocks' rows (one for 5, 3, 16 tokens)."""
    from mini_engine_b200.engine.replay import TraceReplayer
    name = "A"
    r = helpers.random_requests(zoo.ALL[name][0]["vocab"], (200,), seed=5)[0]
    rp = TraceReplayer(zoo.folder(name), "float32", 256, page_size=16)
    rp.run_step({"step": 0, "entries": [{"id": "x", "tokens": r[:150], "want": [149]}], "end": []})
    for p in range(150, 200):
        rp.run_step({"step": p, "entries": [{"id": "x", "tokens": [r[p]], "want": [0]}], "end": []})
    held = {(g.window, g.every): sum(1 for p in t if p >= 0) for g, t in zip(rp.cache.groups, rp.live["x"].block_tables)}
    assert held[(20, 1)] <= 3 and held[(33, 1)] <= 4 and held[(9, 1)] <= 2
    assert held[(None, 5)] == 3 and held[(None, 3)] == 5 and held[(None, 16)] == 1        # 40, 67 and 13 rows in pages of 16


def _with(name, change):
    """A copy of a model's folder with its configuration and tensors changed by ``change(cfg, tensors)``."""
    cfg, seed, _ = zoo.ALL[name]
    cfg = copy.deepcopy(cfg)
    w = zoo.tensors(cfg, seed)
    change(cfg, w)
    return cfg, zoo.write_folder(cfg, w)


def test_a_far_block_decides_the_logits():
    """Model B's first layer sees every earlier token as a block of one.  With its scale raised tenfold single keys carry the
    weight, often hundreds of tokens back: an engine that lost or misplaced far blocks (a page's edge, a block table's row)
    would be wrong by far more than rounding.  The latent layer behind it has no window and is sharpened the same way."""
    def change(cfg, w):
        cfg["layers"][0]["mixer"]["scale"] *= 10.0
        cfg["layers"][1]["mixer"]["scale"] *= 6.0
    cfg, folder = _with("B", change)
    r = helpers.random_requests(cfg["vocab"], (420,), seed=31)[0]
    for steps, tag in ((helpers.trace_whole([r]), "w"), (helpers.trace_decode_tail([r], tail=40), "d"),
                       (helpers.trace_portions([r], sizes=(50, 2, 130, 7)), "p")):
        got, _ = _replay("B", "float32", steps, folder=folder, poison=True)
        _check("B", "float32", [r], got, tag, folder=folder, cfg=cfg, tol=2e-4)


def test_sharp_scores_at_the_edges_of_windows_and_blocks():
    """Model A with every mixer's scale raised eightfold (normed queries and keys bound a score, so the scale is what sharpens
    the softmax): single keys and single blocks carry the weight, and a key one token inside or outside a window, or a block
    that is seen one token too early or too late, changes a position's logits by far more than rounding."""
    def change(cfg, w):
        for layer in cfg["layers"]:
            layer["mixer"]["scale"] *= 8.0
    cfg, folder = _with("A", change)
    reqs = helpers.random_requests(cfg["vocab"], (131, 77), seed=33)
    for steps, tag in ((helpers.trace_whole(reqs), "w"), (helpers.trace_decode_tail(reqs, tail=70), "d"),
                       (helpers.trace_portions(reqs, sizes=(19, 2, 24, 1, 20, 3, 47)), "p")):
        got, _ = _replay("A", "float32", steps, folder=folder, poison=True)
        _check("A", "float32", reqs, got, tag, folder=folder, cfg=cfg, tol=2e-4)


def test_blocks_matter():
    """The same weights with the blocks taken out of the configuration give other logits from the first position on at which a
    block is seen, and the same before it: the engine does look at the blocks, and only where it should."""
    def change(cfg, w):
        for layer in cfg["layers"]:
            layer["mixer"].get("mask", {}).pop("pool", None)
    cfg, folder = _with("A", change)
    r = helpers.random_requests(cfg["vocab"], (90,), seed=35)[0]
    got, _ = _replay("A", "float32", helpers.trace_whole([r]), folder=folder)
    _check("A", "float32", [r], got, "w", folder=folder, cfg=cfg)
    with_blocks = _plain_logits("A", r)
    err = _error(got["w0"], with_blocks)
    first_seen = min(l["mixer"]["mask"]["size"] + l["mixer"]["mask"]["pool"] - 1
                     for l in zoo.ALL["A"][0]["layers"] if l["type"] == "attention")
    assert err[:first_seen].max() < 1e-5 and err[first_seen:].max() > 1e-2


def test_the_correction_steers_the_choice_and_not_the_weights():
    """Corrections of +-3 decide which experts run whatever the scores say; the weights stay the plain sigmoids."""
    def change(cfg, w):
        for i, layer in enumerate(cfg["layers"]):
            if layer["mlp"]:
                E = layer["mlp"]["router"]["experts"]
                w[f"l{i}.mlp.correction"] = (3.0 * (-1.0) ** torch.arange(E)).to(torch.bfloat16)
    cfg, folder = _with("A", change)
    r = helpers.random_requests(cfg["vocab"], (60,), seed=39)[0]
    for steps, tag in ((helpers.trace_whole([r]), "w"), (helpers.trace_decode_tail([r], tail=20), "d")):
        got, _ = _replay("A", "float32", steps, folder=folder, poison=True)
        _check("A", "float32", [r], got, tag, folder=folder, cfg=cfg)
    assert _error(got["d0"], _plain_logits("A", r)).max() > 1e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_one_size_replayed_from_a_graph(dtype):
    """Four portions of 130 tokens with one wanted place each: the shape comes again, so the engine records the step and
    replays it, at other positions each time (a rotation, a mask or a block taken from the recording's positions would show)."""
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
    cfg, w = plain_galupel.load_folder(zoo.folder(name))
    ids = list(prompt)
    for _ in range(n):
        logits = plain_galupel.forward(cfg, w, ids)[-1]
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
