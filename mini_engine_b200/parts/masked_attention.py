"""Grouped-query attention with a mask, a learned sink in the softmax, and choices around the rotation.

q = W_q h, k = W_k h, v = W_v h, each with a bias when ``bias`` is set (then the output projection has one too).  Every q
and k head may be RMS-normed: ``qk_norm`` "before" (with a weight of ``dim`` values for q and one for k, shared by the
heads, in front of the rotation) or "after" (no weight, behind the rotation).  The rotation pairs element i with element
i + rotary_dim / 2 on the first ``rotary_dim`` elements of a head (a ``FrequencyRotary``, whose frequencies may be
rescaled).  score = q . k * scale, then, with ``softcap`` c, c tanh(score / c).  ``mask``: None (every key j <= p),
("window", size, keep_first): keys with p - j < size or j < keep_first, or ("chunk", size): keys of the query's own
chunk, floor(j / size) = floor(p / size).  The weights are exp(s_j) / (exp(sink_h) + sum exp(s_j)) with a learned number
per head when ``sink`` is set: a term without key or value that is neither scaled nor capped.  Keys have ``dim`` elements
and values ``vdim``; the cache is the engine's usual one (pages of keys and of values) with rows of max(dim, vdim)
elements, and it keeps what the mask can still show: the window (and the first tokens), or the chunk being filled.

Scores, softmax, norms, angles and the rotation are float32; the packed projection returns float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import DiskSource, KVCacheNeed, Mixer, ParamDecl
from .linear import Linear
from .registry import PartSpec, build_part, register_mixer


class MaskedSinkAttention(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float, norm_eps: float,
                 position_encoding: Optional[PartSpec | object] = None, qk_norm: Optional[str] = None, bias: bool = False,
                 softcap: Optional[float] = None, mask: Optional[tuple] = None, sink: bool = True):
        super().__init__()
        if num_heads < 1 or num_kv_heads < 1 or num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are no multiple of {num_kv_heads} kv heads")
        if qk_norm not in (None, "before", "after"):
            raise ValueError(f"qk_norm must be None, 'before' or 'after', got {qk_norm!r}")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.dim, self.vdim = dim, vdim
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.qk_norm, self.has_bias, self.has_sink = qk_norm, bias, sink
        self.softcap = float(softcap) if softcap else None
        self.window, self.keep_first, self.chunk = None, 0, None
        if mask is not None:
            if mask[0] == "window" and int(mask[1]) >= 1:
                self.window, self.keep_first = int(mask[1]), int(mask[2]) if len(mask) > 2 and mask[2] else 0
            elif mask[0] == "chunk" and int(mask[1]) >= 1:
                self.chunk = int(mask[1])
            else:
                raise ValueError(f"mask must be ('window', size, keep_first) or ('chunk', size), got {mask!r}")
        if isinstance(position_encoding, PartSpec):
            position_encoding = build_part("position_encoding", position_encoding)
        self.rope = position_encoding
        if self.rope is not None and (self.rope.layout != "half_split" or not hasattr(self.rope, "freq") or self.rope.rotary_dim > dim):
            raise ValueError("MaskedSinkAttention rotates halves of at most dim elements from a table of frequencies "
                             f"(got layout {self.rope.layout!r}, {self.rope.rotary_dim} of {dim})")
        H, G = num_heads, num_kv_heads
        self.pieces = [("q", H * dim), ("k", G * dim), ("v", G * vdim)]
        self.channels = sum(n for _, n in self.pieces)
        self.in_proj = Linear(hidden_size, self.pieces, name="in_proj")
        self.o_proj = Linear(H * vdim, [("o", hidden_size)], name="o")
        self.defer_output_bias = False        # a block that adds the output bias itself (with the residual sum) sets this

    def sub_parts(self):
        parts = [("", self.in_proj), ("", self.o_proj)]
        if self.rope is not None:
            parts.append(("rot.", self.rope))
        return parts

    def param_decls(self):
        decls = []
        if self.has_bias:
            sources, start = [], 0
            for piece, n in self.pieces:
                sources.append(DiskSource(piece + ".b", start, n))
                start += n
            decls += [ParamDecl("in_bias", (self.channels,), sources=sources, role="vector"),
                      ParamDecl("o.b", (self.hidden_size,), role="vector")]
        if self.qk_norm == "before":
            decls += [ParamDecl("q.norm", (self.dim,), init="norm", role="vector"), ParamDecl("k.norm", (self.dim,), init="norm", role="vector")]
        if self.has_sink:
            decls.append(ParamDecl("sink", (self.num_heads,), role="vector"))
        return decls

    def cache_needs(self):
        return [KVCacheNeed(self.num_kv_heads, max(self.dim, self.vdim), self.window, keep_first=self.keep_first, chunk=self.chunk)]

    def first_weight(self):
        return self.in_proj.weight

    def output_bias(self):
        """The output projection's bias when the caller has asked to add it itself (``defer_output_bias``), else None."""
        return self.p("o.b") if self.has_bias and self.defer_output_bias else None

    def forward(self, x, ctx, call):
        H, G, D, V = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        proj = self.in_proj.forward(x, ctx, "attn_proj", out_dtype=torch.float32)
        T = proj.shape[0]
        kv = ctx.kv_cache(call.cache_slot)
        q = ctx.buffer("attn_q", (T, H * D), ctx.act_dtype)
        before = self.qk_norm == "before"
        ops.attn_prep(proj, self.p("in_bias") if self.has_bias else None, self.p("q.norm") if before else None,
                      self.p("k.norm") if before else None, self.qk_norm, self.norm_eps,
                      self.rope.freq if self.rope is not None and self.rope.rotary_dim else None, ctx.positions,
                      kv.slot_mapping if call.writes_cache else None, q, kv.pool, kv.page_size, H, G, D, V)
        out = ctx.buffer("attn_out", (T, H * V), ctx.act_dtype)
        ops.sink_attention(q, None, out, kv.pool, kv.page_size, kv.block_tables, ctx.attn_meta, H, G, D, V, self.scale,
                           self.window, False, sinks=self.p("sink") if self.has_sink else None, softcap=self.softcap,
                           keep_first=self.keep_first, chunk=self.chunk)
        y = self.o_proj.forward(out, ctx, "mixer_out")
        if self.has_bias and not self.defer_output_bias:
            ops.add_row_vector(y, self.p("o.b"))
        return y


register_mixer("masked_sink_attention", MaskedSinkAttention)
