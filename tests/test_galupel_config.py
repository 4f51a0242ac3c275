"""Galupel's configuration, plan and cache bookkeeping on the CPU: what is read, what is refused, which tensors the model asks
for, how many pages a request holds."""
import copy

import pytest

import galupel_models as zoo
from mini_engine_b200.cache.manager import CacheHolder, CacheManager, GroupSpec
from mini_engine_b200.config.model_config import ConfigError, GalupelConfig
from mini_engine_b200.config.registry import get_architecture
from mini_engine_b200.engine.model_runner import plan_cache_groups
from mini_engine_b200.weights.loader import expected_disk_tensors
from mini_engine_b200.weights.random_init import build_model_from_config_dict


@pytest.mark.parametrize("name", sorted(zoo.ALL))
def test_the_model_asks_for_the_designs_tensors(name):
    cfg, seed, _ = zoo.ALL[name]
    _, model = build_model_from_config_dict(cfg)
    want = {k: tuple(v.shape) for k, v in zoo.tensors(cfg, seed).items()}
    got = {k: tuple(e.shape) for k, e in expected_disk_tensors(model).items() if not e.optional}
    assert got == want
    # a second norm of a layer without feed-forward is accepted when a file holds it, and never missed
    extra = {k for k, e in expected_disk_tensors(model).items() if e.optional}
    assert extra == {f"l{i}.norm2" for i, layer in enumerate(cfg["layers"]) if layer["mlp"] is None}


def test_every_number_comes_from_the_file():
    c = GalupelConfig.from_dict(zoo.A)
    assert (c.vocab_size, c.hidden_size, c.norm_eps, c.norm_groups, c.logit_scale, c.logit_softcap) == (101, 48, 1e-6, 3, 0.7, 9.0)
    plan = get_architecture("Galupel").plan(c)
    m0, m1, m2, m3, m4 = (plan.blocks[i].mixer.args for i in range(5))
    assert (m0["num_heads"], m0["num_kv_heads"], m0["dim"], m0["vdim"], m0["window"], m0["pool"]) == (4, 2, 16, 24, 20, 5)
    assert m0["own_kv"] and m0["cache_window"] == 20                      # the widest of 20, 7, 11 and of the blocks 5, 3, 16
    assert (m2["own_kv"], m2["window"], m2["pool"]) == (False, 7, 3) and (m4["window"], m4["pool"]) == (11, 16)
    assert (m1["kv_rank"], m1["rot_dim"], m1["window"], m1["sink"], m1["gate"]) == (24, 8, 33, False, False)
    assert plan.shared[m1["position_encoding"].key].args == {"rotary_dim": 4, "theta": 500.0}
    assert m3["window"] == 9
    assert [c.kv_slot for c in plan.schedule] == [None, None, 0, None, 0]
    f0 = plan.blocks[0].feed_forward.args
    assert (f0["num_experts"], f0["top"], f0["expert_size"], f0["groups"], f0["routing"], f0["activation"]) == (6, 2, 40, (3, 2), "sigmoid_groups", "gelu")
    assert plan.blocks[1].feed_forward.args["groups"] == (1, 1) and plan.blocks[2].feed_forward is None
    assert plan.tie_word_embeddings and plan.embed_norm.args["groups"] == 3 and plan.final_norm.args["param"] == "final.norm"
    assert (plan.logit_scale, plan.logit_softcap) == (0.7, 9.0)
    b = GalupelConfig.from_dict(zoo.B)
    assert (b.norm_groups, b.logit_scale, b.logit_softcap) == (1, 1.0, None)
    pb = get_architecture("Galupel").plan(b)
    assert pb.blocks[1].mixer.args["window"] is None and pb.blocks[4].mixer.args["position_encoding"] is None
    assert pb.blocks[3].mixer.args["pool"] is None and pb.blocks[2].mixer.args["cache_window"] == 13       # blocks of 9, windows of 4 and 13


def test_cache_groups_a_lender_keeps_window_and_block_and_every_reader_has_rows_of_its_own():
    _, model = build_model_from_config_dict(zoo.A)
    groups, location, states = plan_cache_groups(model)
    assert states == {}
    assert [(g.window, g.every, g.planes, g.cache_slots) for g in groups] == [
        (20, 1, 2, (0,)), (None, 5, 2, (0,)), (33, 1, 1, (1,)), (None, 3, 2, (2,)), (9, 1, 1, (3,)), (None, 16, 2, (4,))]
    assert location[0] == (0, 0) and location[(0, "pooled")] == (1, 0) and location[(2, "pooled")] == (3, 0) and 2 not in location
    _, model = build_model_from_config_dict(zoo.C)
    groups, _, _ = plan_cache_groups(model)
    assert [(g.window, g.every, g.num_kv_heads, g.head_dim) for g in groups] == [(128, 1, 2, 64), (None, 16, 2, 64), (100, 1, 1, 192), (None, 32, 2, 64)]


def test_rows_for_blocks_of_tokens_take_pages_by_the_block():
    ps = 4
    m = CacheManager([GroupSpec(10, 1, 8, (0,)), GroupSpec(None, 1, 8, (0,), every=3), GroupSpec(None, 1, 8, (1,), every=7)], 64, ps,
                     enable_prefix_caching=True)
    assert not m.prefix_caching
    h = CacheHolder()
    assert m.allocate(h, 25)
    assert [len(t) for t in h.block_tables] == [7, 3, 1]          # 25 tokens; 9 rows of three tokens; 4 rows of seven
    h.num_computed_tokens = 25
    m.release_behind_window(h)
    assert sum(p >= 0 for p in h.block_tables[0]) == 3 and all(p >= 0 for t in h.block_tables[1:] for p in t)
    assert m.allocate(h, 12)                                      # 37 tokens: 13 rows and 6 rows
    assert [len(t) for t in h.block_tables] == [10, 4, 2]
    h.num_computed_tokens = 37
    m.check([h])
    assert m.fits_at_all(64 * ps) and not m.fits_at_all(64 * ps * 3 + 1, max_portion=8)
    m.free(h)
    assert m.num_free_pages == [64, 64, 64]
    small = CacheManager([GroupSpec(None, 1, 8, (0,), every=2)], 2, ps, enable_prefix_caching=False)
    h = CacheHolder()
    assert small.allocate(h, 16)                                  # 8 rows fill the two pages
    h.num_computed_tokens = 16
    assert not small.allocate(h, 1)                               # the 9th row has none
    assert h.block_tables == [[0, 1]]


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="recurrence"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].pop("mask"), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(pool=0), "positive"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "differ"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4), "groups"),
    (lambda c: c["layers"][3]["mlp"]["router"].update(top=5), "choices"),
    (lambda c: c["norm"].update(groups=5), "norm.groups"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda c: c.pop("width"), "width"),
])
def test_what_cannot_be_is_refused(edit, text):
    cfg = copy.deepcopy(zoo.A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        GalupelConfig.from_dict(cfg)
