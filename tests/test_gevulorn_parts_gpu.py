"""Each mechanism of Gevulorn alone: the kernels behind it against the plain function, on inputs made so that a fault shows."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_gevulorn as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _ops():
    from mini_engine_b200 import ops
    ops.require_extension()
    return ops


def g(seed):
    return torch.Generator().manual_seed(seed)


def _meta(lens, contexts):
    """Step metadata as the kernels read it: requests that bring one token come first."""
    D = sum(1 for n in lens if n == 1)
    assert all(n == 1 for n in lens[:D]) and all(n > 1 for n in lens[D:])
    cu = np.concatenate(([0], np.cumsum(lens))).astype(np.int32)
    lists = {}
    for tq in _ops().ATTN_TILE_SIZES:
        tiles = [(b, q0) for b in range(D, len(lens)) for q0 in range(0, lens[b], tq)]
        lists[tq] = (torch.tensor(tiles or [(0, 0)], dtype=torch.int32, device=DEV), len(tiles))
    return SimpleNamespace(cu_seqlens=torch.tensor(cu, device=DEV), context_lens=torch.tensor(contexts, dtype=torch.int32, device=DEV),
                           num_reqs=len(lens), num_tokens=int(sum(lens)), num_decodes=D, tile_lists=lists,
                           token_req=torch.tensor(np.repeat(np.arange(len(lens)), lens), dtype=torch.int32, device=DEV),
                           max_context_len=max(contexts), num_tiles=sum(n for _, n in lists.values()),
                           workspace=lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=DEV),
                           error_flag=torch.zeros(4, dtype=torch.int32, device=DEV), scratch_context_len=0,
                           typical_context_len=max(contexts))


# ---- gated linear attention ---------------------------------------------------------------------------
PIECES = ("q", "k", "v", "g", "a1")


def _gla_case(H, D, V, rank, tau, seed, W=32, decay_mean=1.0, decay_std=2.0):
    m = {"heads": H, "dim": D, "vdim": V, "tau": tau}
    r = lambda rows, cols, k, s: torch.randn(rows, cols, generator=g(seed + s)) * (k / cols ** 0.5)
    w = {"q": r(H * D, W, 2.0, 1), "k": r(H * D, W, 2.0, 2), "v": r(H * V, W, 1.5, 3), "g": r(H * V, W, 1.5, 4),
         "a1": r(rank, W, 1.5, 5), "a2": r(H * D, rank, 3.0, 6), "a2.b": decay_mean + decay_std * torch.randn(H * D, generator=g(seed + 7)),
         "norm": torch.rand(V, generator=g(seed + 8)) + 0.5, "o": torch.eye(H * V)}
    return m, w


class _GlaRunner:
    """The three launches of the mixer (decays, recurrence, norm and gate) over steps of several requests with state slots."""

    def __init__(self, ops, m, w, slots, eps=1e-5):
        self.ops, self.m, self.w, self.eps = ops, m, w, eps
        H, D, V = m["heads"], m["dim"], m["vdim"]
        self.packed = torch.cat([w[k] for k in PIECES]).to(DEV)
        self.offs, o = {}, 0
        for k in PIECES:
            self.offs[k], o = o, o + w[k].shape[0]
        self.S = torch.full((slots, H, D, V), float("nan"), device=DEV)

    def step(self, rows, lens, contexts, slots, proj=None):
        """rows: the step's inputs [sum(lens), W] in the order of the requests (single tokens first)."""
        ops, m, w = self.ops, self.m, self.w
        H, D, V = m["heads"], m["dim"], m["vdim"]
        T = rows.shape[0]
        proj = (rows.to(DEV) @ self.packed.T).contiguous() if proj is None else proj
        meta = _meta(list(lens), list(contexts))
        la = torch.empty(T, H * D, device=DEV)
        ops.gla_decay(proj, self.offs["a1"], w["a1"].shape[0], w["a2"].to(DEV), w["a2.b"].to(DEV), m["tau"], la)
        runs = ops.gla_chunk_count(meta)
        assert runs >= meta.tile_lists[ops.GLA_CHUNK][1]
        scores = torch.full((T, H, ops.GLA_CHUNK), float("nan"), device=DEV) if runs else None
        states = torch.full((max(runs, 1), H, D, V), float("nan"), device=DEV) if runs else None
        o = torch.full((T, H * V), float("nan"), device=DEV)
        ops.gla_scan(proj, self.offs, la, self.S, meta, torch.tensor(slots, dtype=torch.int32, device=DEV), o, H, D, V, D ** -0.5,
                     scores=scores, chunk_states=states)
        out = torch.empty(T, H * V, device=DEV)
        ops.mlstm_out(o, proj, self.offs["g"], w["norm"].to(DEV), self.eps, out, H, V, shared_weight=True, gate="silu")
        return out.cpu()

    def sequence(self, h, cuts, slot):
        outs, pos = [], 0
        all_proj = h.to(DEV) @ self.packed.T             # once for the whole sequence: a product's rounding may depend on its rows
        for c in cuts:
            outs.append(self.step(h[pos:pos + c], [c], [pos + c], [slot], proj=all_proj[pos:pos + c].contiguous()))
            pos += c
        return torch.cat(outs)


def _plain_gla(h, m, w, eps=1e-5):
    return plain.gla_mixer(h.double(), {"x." + k: v.double() for k, v in w.items()}, "x.", m, eps)[0]


@pytest.mark.parametrize("H, D, V, rank, tau", [(2, 16, 32, 4, 8.0), (3, 24, 40, 3, 2.0), (1, 72, 8, 1, 16.0), (2, 8, 100, 5, 1.0),
                                                (2, 64, 128, 16, 16.0), (1, 130, 70, 2, 4.0)])
def test_gla_against_the_plain_recurrence_and_cut_anywhere(H, D, V, rank, tau):
    ops = _ops()
    T = 200
    m, w = _gla_case(H, D, V, rank, tau, seed=H * 100 + D)
    h = torch.randn(T, 32, generator=g(H + D + V))
    ref = _plain_gla(h, m, w)
    run = _GlaRunner(ops, m, w, slots=3)
    whole = run.sequence(h, [T], slot=1)                                # three runs of 64 tokens and a rest of 8
    assert torch.allclose(whole.double(), ref, atol=3e-4, rtol=1e-3)
    single = run.sequence(h, [1] * T, slot=2)                            # token by token
    assert torch.allclose(single.double(), ref, atol=3e-4, rtol=1e-3)
    cut = run.sequence(h, [2, 1, 30, 2, 64, 1, 65, 35], slot=0)
    assert torch.allclose(cut.double(), ref, atol=3e-4, rtol=1e-3)
    # the state is carried in float32: whole, cut and token by token differ by the order of the sums alone
    assert torch.allclose(whole, single, atol=5e-5, rtol=1e-4) and torch.allclose(whole, cut, atol=5e-5, rtol=1e-4)
    ops.gla_chunks = False
    try:                                                                 # token by token, a token's arithmetic is the same wherever
        assert torch.equal(run.sequence(h, [T], slot=1), single)         # the sequence was cut
    finally:
        ops.gla_chunks = True


def test_gla_requests_of_unequal_length_side_by_side_with_slots_used_again():
    """Two steps of five requests each: single tokens beside portions of 2, 70 and 130 tokens, some from position 0 and some
    that go on from the state an earlier step left; then the slots of finished requests serve new ones from position 0."""
    ops = _ops()
    H, D, V = 3, 24, 40
    m, w = _gla_case(H, D, V, 3, 4.0, seed=77)
    run = _GlaRunner(ops, m, w, slots=5)
    totals = [90, 31, 140, 131, 66]
    hs = [torch.randn(n, 32, generator=g(200 + i)) for i, n in enumerate(totals)]
    refs = [_plain_gla(h, m, w) for h in hs]
    slots = [4, 0, 2, 3, 1]
    first = [89, 30, 70, 1, 64]                       # tokens of the first step; the rest, (1, 1, 70, 130, 2), is the second
    order1 = [3, 0, 1, 2, 4]                          # single tokens first
    out1 = run.step(torch.cat([hs[i][:first[i]] for i in order1]), [first[i] for i in order1], [first[i] for i in order1],
                    [slots[i] for i in order1])
    o = 0
    for i in order1:
        assert torch.allclose(out1[o:o + first[i]].double(), refs[i][:first[i]], atol=3e-4, rtol=1e-3)
        o += first[i]
    order2 = [0, 1, 4, 2, 3]
    lens2 = [totals[i] - first[i] for i in order2]
    out2 = run.step(torch.cat([hs[i][first[i]:] for i in order2]), lens2, [totals[i] for i in order2], [slots[i] for i in order2])
    o = 0
    for i, n in zip(order2, lens2):
        assert torch.allclose(out2[o:o + n].double(), refs[i][first[i]:], atol=3e-4, rtol=1e-3)
        o += n
    # slots 4 and 2 again, from position 0: what they held must not show
    out3 = run.step(torch.cat([hs[2][:100], hs[0][:65]]), [100, 65], [100, 65], [4, 2])
    assert torch.allclose(out3[:100].double(), refs[2][:100], atol=3e-4, rtol=1e-3)
    assert torch.allclose(out3[100:].double(), refs[0][:65], atol=3e-4, rtol=1e-3)


@pytest.mark.parametrize("decay_mean, tau", [(-40.0, 1.0), (40.0, 1.0), (0.0, 0.25)])
def test_gla_decays_that_forget_at_once_or_never(decay_mean, tau):
    """Decays near 0 (a channel forgets everything within a token: exponents far below float32's range inside a run of 64
    tokens) and decays of exactly 1 in float32 (the state only grows): no overflow, no NaN, and the plain result."""
    ops = _ops()
    H, D, V = 2, 16, 24
    m, w = _gla_case(H, D, V, 2, tau, seed=5, decay_mean=decay_mean, decay_std=3.0)
    h = torch.randn(150, 32, generator=g(9))
    ref = _plain_gla(h, m, w)
    run = _GlaRunner(ops, m, w, slots=2)
    for cuts, slot in (([150], 0), ([1] * 150, 1), ([70, 2, 78], 0)):
        got = run.sequence(h, cuts, slot)
        assert torch.isfinite(got).all()
        assert torch.allclose(got.double(), ref, atol=3e-4, rtol=1e-3)


def test_gla_a_slow_channel_carries_the_first_token_across_many_runs():
    """One key channel never decays, and only the first and the last token write to it; the last token's query reads this
    channel alone, so half of its result is the first token's value, carried by the state's walk over six runs of 64 tokens."""
    ops = _ops()
    H, D, V, W = 1, 8, 16, 32
    m, w = _gla_case(H, D, V, 2, 1.0, seed=21)
    w["a2"][:] = 0
    w["a2.b"][:] = -2.0
    w["a2.b"][3] = 60.0                                # channel 3: sigmoid = 1 in float32
    h = torch.randn(401, W, generator=g(22))
    w["k"][3] = 0
    w["q"][:] = 0
    h[:, 0] = 0
    h[0, 0], h[400, 0] = 1.0, 1.0                      # input 0 is set at the first and the last token alone
    w["k"][3, 0] = 5.0                                 # -> k_0[3] = 5, k_t[3] = 0 otherwise
    w["q"][3, 0] = 7.0                                 # -> q_400 = 7 e_3, q_t = 0 otherwise (apart from the first token)
    ref = _plain_gla(h, m, w)
    run = _GlaRunner(ops, m, w, slots=1)
    for cuts in ([401], [300, 101], [400, 1]):
        got = run.sequence(h, cuts, 0)
        assert torch.allclose(got[400].double(), ref[400], atol=1e-4, rtol=1e-4)
    assert ref[400].abs().max() > 0.1


# ---- masked attention with learned sinks -----------------------------------------------------------------
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


def _attention_case(ops, dtype, H, G, D, V, mask, ps, lens, contexts, seed, cap=None, sink_mean=0.5, boost=None, scale=0.37):
    """Runs the kernel on requests whose last ``lens`` tokens are this step's queries; returns (got, reference) per request.
    mask: None, ("window", size, keep_first) or ("chunk", size)."""
    dt = DT[dtype]
    qs = [torch.randn(c, H, D, generator=g(seed + i)) for i, c in enumerate(contexts)]
    ks = [torch.randn(c, G, D, generator=g(seed + 10 + i)) for i, c in enumerate(contexts)]
    vs = [torch.randn(c, G, V, generator=g(seed + 20 + i)) for i, c in enumerate(contexts)]
    sinks = sink_mean + torch.randn(H, generator=g(seed + 30))
    if boost:
        boost(qs, ks)
    qs, ks, vs = ([t.to(dt).float() for t in ts] for ts in (qs, ks, vs))       # what the kernel is given, exactly
    pool, bt = _paged(ks, vs, ps, dt, seed)
    meta = _meta(list(lens), list(contexts))
    q = torch.cat([qq[c - n:].reshape(n, H * D) for qq, n, c in zip(qs, lens, contexts)]).to(dt).to(DEV)
    out = torch.empty(q.shape[0], H * V, dtype=dt, device=DEV)
    window, keep, chunk = None, 0, None
    if mask and mask[0] == "window":
        window, keep = mask[1], mask[2]
        sees = lambda i, j: plain.sees_window(i, j, window, keep)
    elif mask:
        chunk = mask[1]
        sees = lambda i, j: plain.sees_chunk(i, j, chunk)
    else:
        sees = lambda i, j: j <= i
    ops.sink_attention(q, None, out, pool, ps, bt, meta, H, G, D, V, scale, window, False, sinks=sinks.to(DEV), softcap=cap,
                       keep_first=keep, chunk=chunk)
    assert not meta.error_flag.any()
    res, o = [], 0
    for qq, kk, vv, n, c in zip(qs, ks, vs, lens, contexts):
        ref = plain.sink_softmax_attention(qq.double(), kk.double(), vv.double(), scale, sees, sinks.double(), cap)
        res.append((out[o:o + n].float().cpu().double(), ref[c - n:].reshape(n, H * V)))
        o += n
    return res


ATOL = {"float32": 2e-5, "bfloat16": 2e-2}
MASKS = [("window", 40, 3), ("window", 33, 0), ("window", 9, 20), ("window", 1, 1), ("chunk", 24), ("chunk", 64), ("chunk", 1), None]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, D, V, ps, cap", [(4, 2, 16, 24, 16, None), (3, 1, 10, 9, 8, 5.0), (8, 2, 64, 64, 16, 30.0),
                                                 (8, 2, 64, 64, 64, None), (4, 4, 128, 128, 32, 2.0), (6, 2, 40, 40, 16, None),
                                                 (2, 2, 80, 104, 16, 20.0)])
@pytest.mark.parametrize("mask", MASKS, ids=lambda m_: "full" if m_ is None else "-".join(str(x) for x in m_))
def test_attention_in_prompts_and_single_tokens(dtype, H, G, D, V, ps, cap, mask):
    """Single tokens (first in the batch), a prompt from position 0, portions that start in the middle of a page, of a window
    and of a chunk, a portion of two tokens."""
    ops = _ops()
    lens, contexts = (1, 1, 1, 70, 45, 2, 150), (1, 97, 300, 70, 211, 130, 150)
    for (got, ref) in _attention_case(ops, dtype, H, G, D, V, mask, ps, lens, contexts, seed=H * D, cap=cap):
        assert torch.allclose(got, ref, atol=ATOL[dtype], rtol=1e-2 if dtype == "bfloat16" else 1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D, ps", [(16, 16), (64, 16), (64, 64), (40, 8)])
@pytest.mark.parametrize("mask, j_of", [
    (("window", 40, 5), lambda p: p - 39), (("window", 40, 5), lambda p: p - 40),            # last inside, first outside
    (("window", 40, 5), lambda p: 4), (("window", 40, 5), lambda p: 5),                      # last kept, first not kept
    (("window", 128, 70), lambda p: 69), (("window", 128, 70), lambda p: 70),                # kept tokens beyond a page
    (("chunk", 48), lambda p: p // 48 * 48), (("chunk", 48), lambda p: p // 48 * 48 - 1),    # first of the chunk, last before
    (("chunk", 64), lambda p: p // 64 * 64), (("chunk", 64), lambda p: p // 64 * 64 - 1)],
    ids=["win_in", "win_out", "kept_in", "kept_out", "kept_far_in", "kept_far_out", "chunk_in", "chunk_out", "chunk64_in", "chunk64_out"])
def test_one_sharp_key_at_every_edge(dtype, D, ps, mask, j_of):
    """One key gets a score far above the others, just inside or just outside an edge of the mask: either nearly all the weight
    goes to its value or it is not seen at all, for a single token and inside a prompt's portion."""
    ops = _ops()
    H, G, V = 2, 1, D
    lens, contexts = (1, 60), (331, 331)

    def boost(qs, ks):
        for r, (qq, kk) in enumerate(zip(qs, ks)):
            p = qq.shape[0] - 1 - 50 * r                        # the decoded token; a token inside the other request's portion
            kk[j_of(p)] = qq[p, 0:1] * (30.0 / 0.37) / (qq[p, 0] ** 2).sum()
    for (got, ref) in _attention_case(ops, dtype, H, G, D, V, mask, ps, lens, contexts, seed=11 + D, boost=boost):
        assert torch.allclose(got, ref, atol=ATOL[dtype], rtol=1e-2 if dtype == "bfloat16" else 1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D", [16, 64])
def test_a_large_sink_takes_the_weight_and_is_neither_scaled_nor_capped(dtype, D):
    """Sinks of about 9 with capped scores of at most 2: were the sink capped or scaled too, the keys would keep most of the
    weight; as it is the output is nearly nothing."""
    ops = _ops()
    for (got, ref) in _attention_case(ops, dtype, 4, 2, D, D, ("chunk", 32), 16, (1, 50), (77, 120), seed=3, cap=2.0, sink_mean=9.0):
        assert torch.allclose(got, ref, atol=ATOL[dtype], rtol=1e-2 if dtype == "bfloat16" else 1e-5)
        assert got.abs().max() < 0.05


# ---- between the projection and the attention -----------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, D, V, rot, norm, bias, scaling", [
    (4, 2, 16, 24, 8, "after", False, None), (3, 1, 10, 9, 10, "before", True, (4.0, 1.0, 4.0, 64)),
    (2, 2, 64, 64, 32, "before", True, (8.0, 1.0, 4.0, 512)), (6, 2, 40, 40, 40, "after", False, None),
    (2, 1, 12, 20, 0, None, True, None), (1, 1, 8, 8, 8, None, False, None)])
def test_bias_norms_rotation_and_cache_write(dtype, H, G, D, V, rot, norm, bias, scaling):
    """Far positions (the angle is reduced before its sine), rows written to shuffled cache places, values untouched."""
    ops = _ops()
    dt, T, ps, eps = DT[dtype], 37, 8, 1e-5
    C = H * D + G * (D + V)
    proj = torch.randn(T, C + 5, generator=g(1)) * 2                       # columns beyond q|k|v belong to someone else
    b = torch.randn(C, generator=g(2)) if bias else None
    qw, kw = torch.rand(D, generator=g(3)) + 0.5, torch.rand(D, generator=g(4)) + 0.5
    positions = torch.tensor([0, 1, 2, 3, 70001, 1 << 20] + list(range(500, 500 + T - 6)), dtype=torch.int32)
    freqs = plain.rotary_frequencies(rot, 5000.0, dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None) if rot else []
    x = proj[:, :C].double() + (b.double() if bias else 0)
    q, k, v = x[:, :H * D].view(T, H, D), x[:, H * D:H * D + G * D].view(T, G, D), x[:, H * D + G * D:].view(T, G, V)
    if norm == "before":
        q, k = plain.unit_rms(q, eps) * qw.double(), plain.unit_rms(k, eps) * kw.double()
    if rot:
        q, k = plain.rotate_halves(q, positions, freqs), plain.rotate_halves(k, positions, freqs)
    if norm == "after":
        q, k = plain.unit_rms(q, eps), plain.unit_rms(k, eps)
    HD = max(D, V)
    pool = torch.zeros(8, 2, G, ps, HD, dtype=dt, device=DEV)
    slots = torch.randperm(8 * ps, generator=g(5))[:T].to(torch.int32)
    q_out = torch.empty(T, H * D, dtype=dt, device=DEV)
    ops.attn_prep(proj.to(DEV), b.to(DEV) if bias else None, qw.to(DEV) if norm == "before" else None,
                  kw.to(DEV) if norm == "before" else None, norm, eps,
                  torch.tensor(freqs, dtype=torch.float64, device=DEV) if rot else None, positions.to(DEV), slots.to(DEV), q_out,
                  pool, ps, H, G, D, V)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == "float32" else dict(atol=2e-2, rtol=1e-2)
    assert torch.allclose(q_out.float().cpu().double().view(T, H, D), q, **tol)
    rows = pool.float().cpu().double()
    for t in range(T):
        page, off = int(slots[t]) // ps, int(slots[t]) % ps
        assert torch.allclose(rows[page, 0, :, off, :D], k[t], **tol) and torch.allclose(rows[page, 1, :, off, :V], v[t], **tol)


# ---- the residual sum with two layer norms, the activation, the cap -----------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W", [40, 52, 328, 1030, 4100])
def test_residual_sum_and_two_layer_norms(dtype, W):
    """x <- x + mixer + feed-forward + bias + pass vector, then both norms of the same x; a large common offset shows a
    variance that is not taken around the mean."""
    ops = _ops()
    dt, T, eps = DT[dtype], 9, 1e-6
    x = torch.randn(T, W, generator=g(W)) + 30.0
    ya, yb = (torch.randn(T, W, generator=g(W + i)).to(dt) for i in (1, 2))
    va, vb = torch.randn(W, generator=g(W + 3)), torch.randn(W, generator=g(W + 4))
    w1, b1, w2, b2 = (torch.randn(W, generator=g(W + 5 + i)) for i in range(4))
    xd = x.double() + ya.double() + yb.double() + va.double() + vb.double()
    res = x.to(DEV)
    o1, o2 = torch.empty(T, W, dtype=dt, device=DEV), torch.empty(T, W, dtype=dt, device=DEV)
    ops.parallel_norm(res, [ya.to(DEV), yb.to(DEV)], [va.to(DEV), vb.to(DEV)], eps, (w1.to(DEV), b1.to(DEV)), o1, (w2.to(DEV), b2.to(DEV)), o2)
    tol = dict(atol=2e-4, rtol=1e-4) if dtype == "float32" else dict(atol=3e-2, rtol=1e-2)
    assert torch.allclose(res.cpu().double(), xd, atol=1e-5)
    assert torch.allclose(o1.float().cpu().double(), plain.layer_norm(xd, w1.double(), b1.double(), eps), **tol)
    assert torch.allclose(o2.float().cpu().double(), plain.layer_norm(xd, w2.double(), b2.double(), eps), **tol)
    # one norm, nothing added, chosen rows only: the stream stays as it is
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    o3 = torch.empty(3, W, dtype=dt, device=DEV)
    before = res.clone()
    ops.parallel_norm(res, [], [], eps, (w1.to(DEV), b1.to(DEV)), o3, rows=rows)
    assert torch.equal(res, before)
    assert torch.allclose(o3.float().cpu().double(), plain.layer_norm(xd[[7, 0, 3]], w1.double(), b1.double(), eps), **tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_squared_relu_and_the_cap(dtype):
    ops = _ops()
    dt = DT[dtype]
    x = (torch.randn(13, 70, generator=g(1)) * 3).to(dt)
    out = torch.empty(13, 70, dtype=dt, device=DEV)
    ops.activation(x.to(DEV), out, "relu_squared")
    ref = torch.relu(x.double()) ** 2
    assert torch.allclose(out.float().cpu().double(), ref, atol=1e-6 if dtype == "float32" else 0, rtol=1e-6 if dtype == "float32" else 8e-3)
    z = torch.randn(5, 33, generator=g(2)) * 40
    zd = z.to(DEV)
    ops.soft_cap(zd, 15.0)
    assert torch.allclose(zd.cpu().double(), plain.soft_cap(z.double(), 15.0), atol=2e-5)
    assert zd.abs().max() <= 15.0
