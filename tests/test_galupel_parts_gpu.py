"""Each mechanism of Galupel alone: the kernels behind it against the plain function, on inputs made so that a fault shows."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_galupel as plain

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
                           max_context_len=max(contexts), num_tiles=sum(n for _, n in lists.values()),
                           workspace=lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=DEV),
                           error_flag=torch.zeros(4, dtype=torch.int32, device=DEV), scratch_context_len=0,
                           typical_context_len=max(contexts))


# ---- the norm in groups ---------------------------------------------------------------------------------
@pytest.mark.parametrize("W, groups", [(48, 3), (50, 1), (64, 64), (4096, 4), (3000, 8)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_group_norm_adds_normalises_in_place_and_gathers(W, groups, dtype):
    ops, T, eps = _ops(), 9, 1e-5
    x = torch.randn(T, W, generator=g(W)) * 3.0
    y = (torch.randn(T, W, generator=g(W + 1)) * torch.logspace(-2, 2, W)).to(DT[dtype])       # parts of very different size
    w = torch.rand(W, generator=g(W + 2)) + 0.5
    tol = 2e-6 if dtype == "float32" else 1e-2
    res, copy = x.clone().to(DEV), torch.empty(T, W, dtype=DT[dtype], device=DEV)
    ops.group_norm(res, y.to(DEV), w.to(DEV), groups, eps, copy)
    ref = x.double() + plain.group_norm(y.double(), w.double(), groups, eps)
    assert (res.cpu().double() - ref).abs().max() < 2e-5 * ref.abs().max()
    assert (copy.cpu().double() - ref).abs().max() < tol * ref.abs().max()
    res = x.clone().to(DEV)
    ops.group_norm(res, None, w.to(DEV), groups, eps, None)
    ref = plain.group_norm(x.double(), w.double(), groups, eps)
    assert (res.cpu().double() - ref).abs().max() < 2e-6 * ref.abs().max()
    rows = torch.tensor([7, 0, 3, 3], dtype=torch.int32, device=DEV)
    res, out = x.clone().to(DEV), torch.empty(4, W, dtype=DT[dtype], device=DEV)
    ops.group_norm(res, None, w.to(DEV), groups, eps, out, rows=rows)
    assert torch.equal(res.cpu(), x)                                                       # the stream is left alone
    assert (out.cpu().double() - ref[[7, 0, 3, 3]]).abs().max() < tol * ref.abs().max()


# ---- routing --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E, top, count, keep", [(8, 2, 4, 2), (12, 3, 3, 2), (64, 6, 8, 4), (5, 2, 5, 3), (6, 6, 2, 2), (7, 3, 1, 1),
                                                 (16, 1, 16, 1), (40, 5, 2, 1)])
def test_grouped_routing_against_the_plain_rule(E, top, count, keep):
    ops, T = _ops(), 300
    z = torch.randn(T, E, generator=g(E)) * 2.0
    corr = torch.randn(E, generator=g(E + 1)) * 0.5
    for shift in (0.0, -3.0):                       # with -3 every choice score is negative: a group left out must not win as "0"
        c = corr + shift
        idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
        wgt = torch.empty(T, top, dtype=torch.float32, device=DEV)
        ops.moe_route_grouped(z.to(DEV), c.to(DEV), top, count, keep, idx, wgt)
        ref_idx, ref_w = plain.route(z.double(), c.double(), top, count, keep)
        # rows whose decisions are not within rounding of a tie
        s = torch.sigmoid(z.double()) + c.double()
        gaps = (s[:, :, None] - s[:, None, :]).abs() + torch.eye(E) * 9
        clear = gaps.amin((1, 2)) > 1e-5
        assert clear.float().mean() > 0.9
        mine = torch.sort(idx.cpu().long(), 1)
        assert torch.equal(mine.values[clear], torch.sort(ref_idx, 1).values[clear])
        mine_w = torch.zeros(T, E, dtype=torch.float64).scatter_(1, idx.cpu().long(), wgt.cpu().double())
        ref_full = torch.zeros(T, E, dtype=torch.float64).scatter_(1, ref_idx, ref_w)
        assert (mine_w - ref_full)[clear].abs().max() < 1e-6                               # the plain sigmoid, correction left out


def test_routing_and_grouping_of_a_small_step_in_one_kernel():
    ops = _ops()
    for T, E, top, count, keep in ((20, 12, 3, 3, 2), (1, 8, 4, 2, 1), (64, 16, 2, 4, 2)):
        z = torch.randn(T, E, generator=g(T)) * 2.0
        corr = torch.randn(E, generator=g(T + 1)) * 0.5
        mk = lambda *shape, dt=torch.int32: torch.empty(*shape, dtype=dt, device=DEV)
        idx0, w0 = mk(T, top), mk(T, top, dt=torch.float32)
        ops.moe_route_grouped(z.to(DEV), corr.to(DEV), top, count, keep, idx0, w0)
        idx, w, counts, offsets, order, place = mk(T, top), mk(T, top, dt=torch.float32), mk(E), mk(E + 1), mk(T * top), mk(T * top)
        ops.moe_route_grouped_sort(z.to(DEV), corr.to(DEV), top, count, keep, idx, w, counts, offsets, order, place)
        assert torch.equal(idx, idx0) and torch.equal(w, w0)
        flat, off = idx.cpu().reshape(-1), offsets.cpu()
        assert off[0] == 0 and off[-1] == T * top
        for e in range(E):
            pairs = order.cpu()[off[e]:off[e + 1]]
            assert torch.equal(pairs, torch.nonzero(flat == e).reshape(-1).to(torch.int32))        # token order inside an expert
        assert torch.equal(order.cpu()[place.cpu().long()], torch.arange(T * top, dtype=torch.int32))


@pytest.mark.parametrize("T, W, F", [(40, 48, 24), (400, 64, 96)])       # (800 pairs: bfloat16 takes the tcgen05 product)
def test_expert_products_with_the_exact_gelu(T, W, F):
    ops = _ops()
    E, top = 4, 2
    x = torch.randn(T, W, generator=g(1))
    w = torch.randn(E, F, W, generator=g(2)) * 0.3
    idx = torch.stack([torch.randperm(E, generator=g(10 + t))[:top] for t in range(T)]).to(torch.int32)
    for dtype, tol in (("float32", 1e-5), ("bfloat16", 2e-2)):
        dt = DT[dtype]
        counts = torch.empty(E, dtype=torch.int32, device=DEV)
        offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
        order = torch.empty(T * top, dtype=torch.int32, device=DEV)
        place = torch.empty(T * top, dtype=torch.int32, device=DEV)
        ops.moe_sort(idx.to(DEV), E, counts, offsets, order, place)
        out = torch.empty(T * top, F, dtype=dt, device=DEV)
        err = torch.zeros(4, dtype=torch.int32, device=DEV)
        ops.moe_gemm(x.to(DEV).to(dt), order, top, w.to(DEV).to(dt), offsets, out, activation="gelu", err=err,
                     workspace=lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=DEV))
        assert int(err.abs().sum()) == 0
        xr, wr = x.to(dt).double(), w.to(dt).double()
        for t in range(0, T, max(1, T // 40)):
            for k in range(top):
                ref = torch.nn.functional.gelu(xr[t] @ wr[idx[t, k]].T)
                got = out[place[t * top + k]].cpu().double()
                assert (got - ref).abs().max() < tol * max(1.0, ref.abs().max())


def test_scaled_and_capped_logits():
    ops = _ops()
    z = torch.randn(5, 77, generator=g(3)) * 40
    for cap, scale in ((30.0, 0.5), (None, 0.25), (2.0, 1.0)):
        x = z.clone().to(DEV)
        ops.soft_cap(x, cap, scale)
        ref = z.double() * scale
        ref = cap * torch.tanh(ref / cap) if cap else ref
        assert (x.cpu().double() - ref).abs().max() < 1e-5 * max(1.0, float(ref.abs().max()))


# ---- a window and pooled blocks ---------------------------------------------------------------------------
class _Caches:
    """The token cache and the cache of pooled blocks of a few requests, pages scattered over the pools."""

    def __init__(self, ops, dtype, G, D, Dv, page, P, lengths, seed):
        self.ops, self.G, self.D, self.Dv, self.page, self.P = ops, G, D, Dv, page, P
        HD = max(D, Dv)
        n_pages = sum((n + page - 1) // page for n in lengths) + 3
        perm = torch.randperm(n_pages, generator=g(seed)).tolist()
        self.pool = torch.full((n_pages, 2, G, page, HD), float("nan"), dtype=DT[dtype], device=DEV)
        self.pooled = torch.full((n_pages, 2, G, page, HD), float("nan"), dtype=DT[dtype], device=DEV)
        width = max((n + page - 1) // page for n in lengths)
        self.bt = torch.full((len(lengths), width), -1, dtype=torch.int32)
        self.pbt = torch.full((len(lengths), width), -1, dtype=torch.int32)
        for b, n in enumerate(lengths):
            for i in range((n + page - 1) // page):
                self.bt[b, i] = perm.pop()
            for i in range(((n + P - 1) // P + page - 1) // page):
                self.pbt[b, i] = (self.bt[b, i] + 1) % n_pages      # any pages do: the pools are separate
        self.k = [torch.randn(n, G, D, generator=g(seed + 10 + b)).to(DT[dtype]) for b, n in enumerate(lengths)]
        self.v = [torch.randn(n, G, Dv, generator=g(seed + 20 + b)).to(DT[dtype]) for b, n in enumerate(lengths)]
        for b, n in enumerate(lengths):
            for j in range(n):
                pg, off = int(self.bt[b, j // page]), j % page
                self.pool[pg, 0, :, off, :D] = self.k[b][j].to(DEV)
                self.pool[pg, 1, :, off, :Dv] = self.v[b][j].to(DEV)
        self.bt, self.pbt = self.bt.to(DEV), self.pbt.to(DEV)
        # the blocks' rows, formed as a step would form them: a token a launch for some, many at once for others
        for b, n in enumerate(lengths):
            pos = torch.arange(n, dtype=torch.int32)
            for lo, hi in ((0, n // 3), (n // 3, n // 3 + 1), (n // 3 + 1, n)):
                if hi - lo > 1 and lo > 0:          # as a step of one request's portion: a launch by completed blocks
                    ops.pool_kv(self.pool, self.bt[b:b + 1], self.pooled, self.pbt[b:b + 1], pos[lo:hi].to(DEV).contiguous(),
                                torch.zeros(hi - lo, dtype=torch.int32, device=DEV), P, D, Dv, page, meta=_meta([hi - lo], [hi]))
                elif hi > lo:                       # a launch by tokens
                    ops.pool_kv(self.pool, self.bt, self.pooled, self.pbt, pos[lo:hi].to(DEV).contiguous(),
                                torch.full((hi - lo,), b, dtype=torch.int32, device=DEV), P, D, Dv, page)

    def plain(self, b, q, heads, scale, window, sharp=None):
        """Outputs [T, heads, Dv] of request b's queries q [T, heads, D] at positions 0 .. T - 1."""
        k, v = self.k[b].double(), self.v[b].double()
        T, P, G = q.shape[0], self.P, self.G
        nb = T // P
        kp, vp = k[:nb * P].reshape(nb, P, G, self.D).mean(1), v[:nb * P].reshape(nb, P, G, self.Dv).mean(1)
        out = torch.zeros(T, heads, self.Dv, dtype=torch.float64)
        for h in range(heads):
            kv = h // (heads // G)
            at, ab = plain.pooled_window_weights(q[:, h].double() @ k[:T, kv].T * scale, q[:, h].double() @ kp[:, kv].T * scale, window, P)
            out[:, h] = at @ v[:T, kv] + ab @ vp[:, kv]
        return out


CASES = [  # heads, kv heads, dim, vdim, window, block, page
    (4, 2, 16, 24, 20, 5, 16), (3, 1, 10, 9, 1, 1, 8), (6, 3, 8, 8, 4, 9, 8), (2, 2, 48, 48, 37, 12, 16),
    (8, 2, 64, 64, 128, 16, 16), (8, 2, 64, 64, 40, 7, 32), (4, 4, 128, 128, 130, 33, 16), (16, 1, 64, 64, 64, 64, 64),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, D, Dv, window, P, page", CASES)
def test_window_and_pooled_blocks_in_prompts_and_single_tokens(H, G, D, Dv, window, P, page, dtype):
    """Queries scaled up so that a row's weight sits on a few keys or blocks: one token or one block more or less in the mask
    shows.  A whole prompt, then single tokens at contexts around every edge (a block just seen and not yet, pages' borders)."""
    ops = _ops()
    lengths = [3 * window + 5 * P + 70, window + P + 3, 9]
    c = _Caches(ops, dtype, G, D, Dv, page, P, lengths, seed=H * 7 + D)
    scale = 6.0 / D ** 0.5
    tol = 2e-5 if dtype == "float32" else 3e-2
    q = [torch.randn(n, H, D, generator=g(50 + b)).to(DT[dtype]) for b, n in enumerate(lengths)]
    refs = [c.plain(b, q[b], H, scale, window) for b in range(len(lengths))]
    # all prompts in one step
    meta = _meta(lengths, lengths)
    qs = torch.cat([x.reshape(x.shape[0], H * D) for x in q]).to(DEV)
    out = torch.full((qs.shape[0], H * Dv), float("nan"), dtype=DT[dtype], device=DEV)
    ops.sink_attention(qs, None, out, c.pool, page, c.bt, meta, H, G, D, Dv, scale, window, False, pooled=(c.pooled, c.pbt, P))
    got = out.cpu().double().reshape(-1, H, Dv)
    ref = torch.cat(refs)
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max() < tol * ref.abs().max(), int(((got - ref).abs().amax((1, 2)) > tol * ref.abs().max()).nonzero()[0])
    # single tokens of request 0 at many contexts, batched with one of request 1
    n0 = lengths[0]
    edges = sorted({p for b in range(n0 // P) for p in (b * P + P - 1 + window - 1, b * P + P - 1 + window, b * P + P + window)
                    if 0 <= p < n0} | {0, 1, window - 1, window, n0 - 1} | set(range(page - 1, n0, page)))
    for p in edges[:40]:
        if p >= n0:
            continue
        meta = _meta([1, 1], [p + 1, lengths[1]])
        bt = torch.stack([c.bt[0], c.bt[1]]).contiguous()
        pbt = torch.stack([c.pbt[0], c.pbt[1]]).contiguous()
        qs = torch.stack([q[0][p].reshape(-1), q[1][-1].reshape(-1)]).to(DEV)
        out = torch.full((2, H * Dv), float("nan"), dtype=DT[dtype], device=DEV)
        ops.sink_attention(qs, None, out, c.pool, page, bt, meta, H, G, D, Dv, scale, window, False, pooled=(c.pooled, pbt, P))
        got = out.cpu().double().reshape(2, H, Dv)
        for mine, want in ((got[0], refs[0][p]), (got[1], refs[1][-1])):
            assert (mine - want).abs().max() < tol * ref.abs().max(), f"a single token at position {p}"


def test_the_pooled_rows_are_the_means_of_what_the_cache_holds():
    ops = _ops()
    c = _Caches(ops, "bfloat16", 2, 16, 24, 8, 5, [43], seed=3)
    for b in range(43 // 5):
        pg, off = int(c.pbt[0, b // 8]), b % 8
        k = c.k[0][b * 5:(b + 1) * 5].float().mean(0)
        v = c.v[0][b * 5:(b + 1) * 5].float().mean(0)
        assert torch.equal(c.pooled[pg, 0, :, off, :16].cpu(), k.to(torch.bfloat16))
        assert torch.equal(c.pooled[pg, 1, :, off, :24].cpu(), v.to(torch.bfloat16))
    assert torch.isnan(c.pooled[int(c.pbt[0, 1]), 0, 0, 0, 0])             # block 8 is not complete at 43 tokens


def test_the_tensor_core_kernels_agree_with_the_cuda_cores():
    """bfloat16 with keys and values of 64: the prompt goes through the tcgen05 kernel and single tokens through the split-K
    kernel, each with the pooled blocks as tiles of their own; with the switch off both run on the CUDA cores."""
    ops = _ops()
    H, G, D, window, P, page = 8, 2, 64, 100, 12, 16
    lengths = [700, 131]
    c = _Caches(ops, "bfloat16", G, D, D, page, P, lengths, seed=11)
    scale = 4.0 / D ** 0.5
    q = [torch.randn(n, H, D, generator=g(60 + b)).to(torch.bfloat16) for b, n in enumerate(lengths)]
    outs = {}
    for fast in (True, False):
        ops.use_sink_attention_mma = fast
        try:
            meta = _meta(lengths, lengths)
            qs = torch.cat([x.reshape(x.shape[0], H * D) for x in q]).to(DEV)
            out = torch.full((qs.shape[0], H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
            before = ops.launches
            ops.sink_attention(qs, None, out, c.pool, page, c.bt, meta, H, G, D, D, scale, window, False, pooled=(c.pooled, c.pbt, P))
            meta = _meta([1, 1], lengths)
            qs = torch.stack([q[0][-1].reshape(-1), q[1][-1].reshape(-1)]).to(DEV)
            one = torch.full((2, H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
            ops.sink_attention(qs, None, one, c.pool, page, c.bt, meta, H, G, D, D, scale, window, False, pooled=(c.pooled, c.pbt, P))
            torch.cuda.synchronize()
            assert int(meta.error_flag.abs().sum()) == 0
            outs[fast] = (out.cpu().float(), one.cpu().float())
        finally:
            ops.use_sink_attention_mma = True
    ref = torch.cat([c.plain(b, q[b], H, scale, window) for b in range(2)]).reshape(-1, H * D)
    for fast in (True, False):
        assert (outs[fast][0].double() - ref).abs().max() < 3e-2 * ref.abs().max()
        assert (outs[fast][1][0].double() - ref[699]).abs().max() < 3e-2 * ref.abs().max()
        assert (outs[fast][1][1].double() - ref[-1]).abs().max() < 3e-2 * ref.abs().max()
