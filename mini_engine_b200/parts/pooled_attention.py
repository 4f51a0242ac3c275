"""Grouped-query attention over a sliding window and, behind the window, pooled blocks of tokens.

q = W_q h, k = W_k h, v = W_v h (no biases); every q and k head is RMS-normed with a weight of ``dim`` values that the heads
share (one for q, one for k); positions do not enter the scores.  score = q . k * scale * temp[h] with a learned number per
query head (``head_scale``).  A query at position p sees the keys j with 0 <= p - j < window and, beside them, ONE key and value
for every block of ``pool`` consecutive tokens that lies wholly in front of the window: block b (positions b * pool ..
b * pool + pool - 1) is seen if b * pool + pool - 1 <= p - window, its key is the mean of its tokens' keys as the cache holds
them and its value the mean of their values.  A token that has left the window while its block is not yet seen is not seen at
all.  Tokens and blocks share one softmax.  ``pool`` None: a plain window.

The tokens' keys and values live in the engine's usual pages (rows of max(dim, vdim) elements), of which the cache keeps the
window and at least a block (``cache_window``); the blocks' means live in a second cache of the same layout with one row per
block (``KVCacheNeed(every=pool, name="pooled")``), which is never given back.  A row of it is written in the step that brings
the block's last token.

``own_kv`` False: the mixer has no key and value projections; it reads the token pages of another call (``call.kv_slot``) with
its own queries, window and block size, and keeps pooled rows of its own.  ``cache_window``: what the token pages must keep
for all mixers that read them (the widest of their windows and blocks).

Scores, softmax, norms and the means are float32; the packed projection returns float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import KVCacheNeed, Mixer, ParamDecl
from .linear import Linear
from .registry import register_mixer


class PooledWindowAttention(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float, norm_eps: float,
                 window: int, pool: Optional[int] = None, cache_window: Optional[int] = None, own_kv: bool = True,
                 head_scale: bool = True, out_dtype: Optional[str] = None):
        super().__init__()
        if num_heads < 1 or num_kv_heads < 1 or num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are no multiple of {num_kv_heads} kv heads")
        if window < 1 or (pool is not None and pool < 1):
            raise ValueError(f"a window of {window} tokens with blocks of {pool} cannot be")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.dim, self.vdim = dim, vdim
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.window, self.pool = int(window), int(pool) if pool else None
        self.cache_window = int(cache_window) if cache_window else max(self.window, self.pool or 1)
        self.own_kv, self.has_head_scale = own_kv, head_scale
        self.out_dtype = getattr(torch, out_dtype) if out_dtype else None     # what the output projection returns (None: the working dtype)
        H, G = num_heads, num_kv_heads
        self.pieces = [("q", H * dim)] + ([("k", G * dim), ("v", G * vdim)] if own_kv else [])
        self.in_proj = Linear(hidden_size, self.pieces, name="in_proj")
        self.o_proj = Linear(H * vdim, [("o", hidden_size)], name="o")

    def sub_parts(self):
        return [("", self.in_proj), ("", self.o_proj)]

    def param_decls(self):
        decls = [ParamDecl("q.norm", (self.dim,), init="norm", role="vector")]
        if self.own_kv:
            decls.append(ParamDecl("k.norm", (self.dim,), init="norm", role="vector"))
        if self.has_head_scale:
            decls.append(ParamDecl("temp", (self.num_heads,), init="norm", role="vector"))
        return decls

    def cache_needs(self):
        row = max(self.dim, self.vdim)
        needs = [KVCacheNeed(self.num_kv_heads, row, self.cache_window)] if self.own_kv else []
        if self.pool:
            needs.append(KVCacheNeed(self.num_kv_heads, row, None, every=self.pool, name="pooled"))
        return needs

    def first_weight(self):
        return self.in_proj.weight

    def forward(self, x, ctx, call):
        H, G, D, V = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        proj = self.in_proj.forward(x, ctx, "attn_proj", out_dtype=torch.float32)
        T = proj.shape[0]
        if not self.own_kv and call.kv_slot is None:
            raise ValueError("a mixer without keys and values of its own needs the cache slot of the call that has them (kv_slot)")
        kv = ctx.kv_cache(call.cache_slot if self.own_kv else call.kv_slot)
        writes = self.own_kv and call.writes_cache
        q = ctx.buffer("attn_q", (T, H * D), ctx.act_dtype)
        ops.attn_prep(proj, None, self.p("q.norm"), self.p("k.norm") if self.own_kv else None, "before", self.norm_eps, None,
                      ctx.positions, kv.slot_mapping if writes else None, q, kv.pool, kv.page_size, H, G, D, V,
                      q_scale=self.p("temp") if self.has_head_scale else None, own_kv=self.own_kv)
        pooled = None
        if self.pool:
            pv = ctx.kv_cache(call.cache_slot, "pooled")
            if call.writes_cache:
                ops.pool_kv(kv.pool, kv.block_tables, pv.pool, pv.block_tables, ctx.positions, ctx.token_req, self.pool, D, V,
                            kv.page_size, meta=ctx.attn_meta)
            pooled = (pv.pool, pv.block_tables, self.pool)
        out = ctx.buffer("attn_out", (T, H * V), ctx.act_dtype)
        ops.sink_attention(q, None, out, kv.pool, kv.page_size, kv.block_tables, ctx.attn_meta, H, G, D, V, self.scale,
                           self.window, False, pooled=pooled)
        return self.o_proj.forward(out, ctx, "mixer_out", out_dtype=self.out_dtype)


register_mixer("pooled_window_attention", PooledWindowAttention)
