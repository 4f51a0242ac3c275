"""Gevulorn's configuration, plan and cache bookkeeping, on the CPU."""
import copy
import math

import pytest
import torch

import gevulorn_models as zoo
import plain_gevulorn as plain
from mini_engine_b200.cache.manager import CacheHolder, CacheManager, GroupSpec
from mini_engine_b200.config.model_config import ConfigError, GevulornConfig
from mini_engine_b200.config.registry import get_architecture, load_model_config
from mini_engine_b200.parts import DecoderModel, FrequencyRotary
from mini_engine_b200.parts.base import KVCacheNeed, StateNeed
from mini_engine_b200.weights.loader import WeightsError, expected_disk_tensors, load_weights


def _model(name):
    cfg = load_model_config(zoo.folder(name))
    return cfg, DecoderModel(get_architecture(cfg.architecture).plan(cfg))


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_number_comes_from_the_configuration_and_the_rank_from_the_weights(name):
    raw = zoo.ALL[name][0]
    cfg, model = _model(name)
    assert isinstance(cfg, GevulornConfig) and cfg.vocab_size == raw["vocab"] and cfg.hidden_size == raw["width"]
    assert cfg.embedding_scale == raw["embedding"]["scale"] and cfg.logit_softcap == raw.get("logit_softcap")
    for got, want in zip(cfg.layers, raw["layers"]):
        for k, v in want["mixer"].items():
            assert got["mixer"][k] == v
        if want["type"] == "gla":
            assert got["mixer"]["decay_rank"] == zoo.RANKS[name]
    # the engine wants exactly the tensors the writer wrote
    disk = set(zoo.tensors(raw, 0, zoo.RANKS[name]))
    assert set(expected_disk_tensors(model)) - {n for n in expected_disk_tensors(model) if n.endswith(("norm2", "norm2.b")) and n not in disk} == disk
    load_weights(model, zoo.folder(name), torch.float32, "cpu")
    assert model.head.softcap == raw.get("logit_softcap")


def test_the_order_of_layer_runs_and_their_cache_slots():
    cfg, model = _model("A")                                   # layers 1..3 twice
    assert cfg.layer_runs() == plain.layer_runs(zoo.A) == [(0, None), (1, 0), (2, None), (3, None), (1, 1), (2, None), (3, None), (4, None)]
    calls = model.schedule
    assert [c.block for c in calls] == [0, 1, 2, 3, 1, 2, 3, 4] and [c.cache_slot for c in calls] == list(range(8))
    assert [c.add_row for c in calls] == [None, 0, None, None, 1, None, None, None]
    assert model.slot_needs[1] == model.slot_needs[4] == [KVCacheNeed(2, 24, 20, keep_first=2)]
    assert model.slot_needs[3] == [KVCacheNeed(2, 16, None, chunk=24)]
    assert model.slot_needs[2] == model.slot_needs[5] == [StateNeed((4, 8, 8), "float32", "S")]
    cfg, model = _model("D")                                   # the last layer four times, a state each
    assert [c.block for c in model.schedule] == [0, 1, 2, 2, 2, 2] and [c.add_row for c in model.schedule] == [None, None, 0, 1, 2, 3]
    assert model.pass_vectors.rows == 4
    cfg, model = _model("C")                                   # no loop: no pass vectors
    assert model.pass_vectors is None and all(c.add_row is None for c in model.schedule)


def test_a_loop_over_nothing_is_no_loop_and_one_pass_still_adds_its_vector():
    raw = copy.deepcopy(zoo.B)
    raw["loop"] = {"start": 2, "stop": 2, "times": 5}
    assert GevulornConfig.from_dict(raw).layer_runs() == [(i, None) for i in range(4)]
    raw["loop"] = {"start": 0, "stop": 4, "times": 1}
    assert GevulornConfig.from_dict(raw).layer_runs() == plain.layer_runs(raw) == [(0, 0), (1, None), (2, None), (3, None)]


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("tau"), "tau"),
    (lambda c: c["layers"][1]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][3]["mixer"]["rot"]["scaling"].update(high=0.5), "scaling"),
    (lambda c: c["layers"][3]["mixer"]["mask"].update(keep_first=2), "keep"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "mlp"),
    (lambda c: c.update(loop={"start": 3, "stop": 9, "times": 2}), "loop"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_what_cannot_be_is_refused(change, text):
    raw = copy.deepcopy(zoo.A)
    change(raw)
    with pytest.raises(ConfigError, match=text):
        GevulornConfig.from_dict(raw)


def test_absent_keys_mean_absent_mechanisms():
    raw = copy.deepcopy(zoo.B)
    del raw["embedding"]
    cfg = GevulornConfig.from_dict(raw)
    assert cfg.embedding_scale == 1.0 and cfg.logit_softcap is None
    for layer in cfg.layers:
        layer["mixer"].setdefault("decay_rank", 3)
    plan = get_architecture("Gevulorn").plan(cfg)
    a2 = plan.blocks[1].mixer.args                            # no chunks, no cap, plain frequencies
    assert a2["mask"] is None and a2["softcap"] is None and plan.shared[a2["position_encoding"].key].args["scaling"] is None
    assert plan.blocks[0].mixer.args["mask"] == ("window", 17, 0)
    assert plan.blocks[2].feed_forward is None
    with pytest.raises(ConfigError, match="rank"):            # without weights and without decay_rank nobody knows the rank
        get_architecture("Gevulorn").plan(GevulornConfig.from_dict(raw))


def test_a_second_norm_without_a_feed_forward_is_accepted_but_not_needed():
    cfg, seed, _ = zoo.ALL["B"]
    w = zoo.tensors(cfg, seed, zoo.RANKS["B"])
    assert "l2.norm2" not in w
    w["l2.norm2"], w["l2.norm2.b"] = torch.ones(52, dtype=torch.bfloat16), torch.zeros(52, dtype=torch.bfloat16)
    folder = zoo.write_folder(cfg, w)
    c = load_model_config(folder)
    load_weights(DecoderModel(get_architecture(c.architecture).plan(c)), folder, torch.float32, "cpu")
    w["l2.norm3"] = w["l2.norm2"].clone()
    folder = zoo.write_folder(cfg, w)
    with pytest.raises(WeightsError) as e:
        load_weights(DecoderModel(get_architecture(c.architecture).plan(c)), folder, torch.float32, "cpu")
    assert e.value.unexpected == ["l2.norm3"] and not e.value.missing


@pytest.mark.parametrize("dims, base, scaling", [(16, 100.0, (4.0, 1.0, 4.0, 64)), (32, 1e6, (8.0, 1.0, 4.0, 512)), (8, 5000.0, None),
                                                 (12, 10.0, (2.0, 0.5, 3.0, 40)), (64, 500000.0, (32.0, 1.0, 4.0, 8192))])
def test_rescaled_frequencies(dims, base, scaling):
    sc = dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None
    got = FrequencyRotary(dims, base, sc).frequencies()
    want = plain.rotary_frequencies(dims, base, sc)
    assert len(got) == dims // 2 and all(math.isclose(a, b, rel_tol=1e-14) for a, b in zip(got, want))
    if sc:                                                      # all three ranges occur in the first and last cases' tables
        plain_f = plain.rotary_frequencies(dims, base, None)
        kinds = {"kept" if a == b else ("divided" if math.isclose(a, b / sc["factor"]) else "between") for a, b in zip(got, plain_f)}
        assert "kept" in kinds and len(kinds) >= 2


def _holder_after(manager, tokens_per_step):
    h = CacheHolder()
    for n in tokens_per_step:
        assert manager.allocate(h, n)
        h.num_computed_tokens += n
        manager.release_behind_window(h)
    return h


def test_a_window_group_keeps_the_pages_of_the_first_tokens():
    ps = 4
    m = CacheManager([GroupSpec(10, 1, 8, (0,), keep_first=6), GroupSpec(10, 1, 8, (1,)), GroupSpec(None, 1, 8, (2,))], 64, ps,
                     enable_prefix_caching=False)
    h = _holder_after(m, [23, 1, 1, 1, 30, 1])
    computed = 57
    kept, plain_window, everything = h.block_tables
    assert all(p >= 0 for p in everything)
    lowest = computed - 10 + 1                                  # the lowest key that a token still to come can see
    for i in range(len(kept)):
        visible = (i + 1) * ps > lowest
        assert (plain_window[i] >= 0) == visible
        assert (kept[i] >= 0) == (visible or i * ps < 6)        # pages 0 and 1 hold tokens 0..5
    m.free(h)
    m.check([])
    assert m.num_free_pages == [64, 64, 64]


def test_a_chunk_group_keeps_the_chunk_that_is_being_filled():
    ps = 4
    m = CacheManager([GroupSpec(None, 1, 8, (0,), chunk=10)], 64, ps, enable_prefix_caching=False)
    h = CacheHolder()
    for n in [7, 2, 1, 1, 5, 3, 1, 12, 1]:
        assert m.allocate(h, n)
        h.num_computed_tokens += n
        m.release_behind_window(h)
        start = h.num_computed_tokens // 10 * 10               # the next token's chunk starts here
        for i, p in enumerate(h.block_tables[0]):
            assert (p >= 0) == ((i + 1) * ps > start), (h.num_computed_tokens, i)
    assert not m.prefix_caching
    m.free(h)
    m.check([])
