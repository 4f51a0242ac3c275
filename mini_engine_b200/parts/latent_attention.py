"""Attention through a low-rank latent of keys and values, over a paged cache of one row per token.

Per head ``dim`` unrotated and ``rot_dim`` rotated query/key dimensions, values of ``vdim``, a latent of ``kv_rank``:
q = W_q h, head by head [unrotated | rotated]; W_dkv h gives kv_rank + rot_dim values, the first kv_rank of them
divided by their root mean square and multiplied by a weight (the latent c), the rest one rotated key part shared by
all heads; a head's unrotated key is W_uk c and its value W_uv c, so only c and the rotated key part are cached (one
cache row of kv_rank + rot_dim values per token).  score = (q_unrotated . k_unrotated + q_rotated . k_rotated) * scale,
causal; with a ``window`` w a query at position p sees the keys p - w < j <= p only, and the cache keeps no more.  Optional: a sink (a learned logit per head that joins the softmax's denominator once, with no key and no
value) and a gate (head h's output times sigmoid(W_g h)_h).

The key up-projection is folded into the query (qa_h = W_uk,h^T q_h) and the value up-projection is applied to the
softmax-weighted sum of latents, so the attention kernel reads the cache rows as they are, for portions of prompts
and for single tokens alike.  Scores, softmax, the latent's norm and the rotation are float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import KVCacheNeed, Mixer, ParamDecl
from .linear import Linear
from .registry import PartSpec, build_part, register_mixer


class LatentAttention(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float,
                 norm_eps: float, position_encoding: Optional[PartSpec | object], sink: bool = True, gate: bool = True,
                 window: Optional[int] = None, out_dtype: Optional[str] = None):
        super().__init__()
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.dim, self.rot_dim, self.vdim, self.kv_rank = dim, rot_dim, vdim, kv_rank
        self.scale = float(scale)
        self.norm_eps = float(norm_eps)
        self.has_sink, self.has_gate = sink, gate
        if window is not None and window < 1:
            raise ValueError(f"LatentAttention: a window of {window} tokens cannot be")
        self.window = int(window) if window else None
        self.out_dtype = getattr(torch, out_dtype) if out_dtype else None     # what the output projection returns (None: the working dtype)
        if isinstance(position_encoding, PartSpec):
            position_encoding = build_part("position_encoding", position_encoding)
        self.rope = position_encoding
        if self.rope is not None and (self.rope.layout != "interleaved" or self.rope.rotary_dim > rot_dim):
            raise ValueError("LatentAttention rotates neighbouring pairs of at most rot_dim elements "
                             f"(got layout {self.rope.layout!r}, {self.rope.rotary_dim} of {rot_dim})")
        H = num_heads
        pieces = [("q", H * (dim + rot_dim)), ("dkv", kv_rank + rot_dim)] + ([("g", H)] if gate else [])
        self.in_proj = Linear(hidden_size, pieces, name="in_proj")
        self.offsets = {"q": 0, "c": H * (dim + rot_dim), "g": H * (dim + rot_dim) + kv_rank + rot_dim}
        self.o_proj = Linear(H * vdim, [("o", hidden_size)], name="o")
        self._uk = self._uv_t = self._no_freq = None

    def sub_parts(self):
        parts = [("", self.in_proj), ("", self.o_proj)]
        if self.rope is not None:
            parts.append(("rot.", self.rope))
        return parts

    def param_decls(self):
        H = self.num_heads
        decls = [ParamDecl("dkv.norm", (self.kv_rank,), init="norm", role="vector"),
                 ParamDecl("uk", (H * self.dim, self.kv_rank)), ParamDecl("uv", (H * self.vdim, self.kv_rank))]
        if self.has_sink:
            decls.append(ParamDecl("sink", (H,), role="vector"))
        return decls

    def cache_needs(self):
        return [KVCacheNeed(1, self.kv_rank + self.rot_dim, self.window, planes=1)]

    def first_weight(self):
        return self.in_proj.weight

    def finalize(self, dtype, device):
        H = self.num_heads
        self._uk = self.p("uk").view(H, self.dim, self.kv_rank)                     # [H, dim, kv_rank]: q -> latent space
        self._uv_t = self.p("uv").view(H, self.vdim, self.kv_rank).transpose(1, 2)  # [H, kv_rank, vdim]
        self._no_freq = torch.zeros(0, dtype=torch.float64, device=device)

    def forward(self, x, ctx, call):
        H, D, R, V, C = self.num_heads, self.dim, self.rot_dim, self.vdim, self.kv_rank
        proj = self.in_proj.forward(x, ctx, "latent_proj", out_dtype=torch.float32)
        T = proj.shape[0]
        kv = ctx.kv_cache(call.cache_slot)
        dt = ctx.act_dtype
        q_plain = ctx.buffer("latent_q_plain", (T, H, D), dt)
        q_rot = ctx.buffer("latent_q_rot", (T, H, R), dt)
        gate = ctx.buffer("latent_gate", (T, H), torch.float32) if self.has_gate else None
        inv_freq = self.rope.inv_freq if self.rope is not None else self._no_freq
        ops.latent_prep(proj, self.offsets, self.p("dkv.norm"), self.norm_eps, inv_freq, inv_freq.numel() * 2, ctx.positions,
                        kv.slot_mapping if call.writes_cache else None, kv.pool, q_plain, q_rot, gate, H, D, R, C)
        q_abs = ctx.buffer("latent_q_abs", (H, T, C), dt)
        ops.batched_heads_mm(q_plain.transpose(0, 1), self._uk, q_abs)
        o_lat = ctx.buffer("latent_o", (H, T, C), dt)
        ops.latent_attention(q_abs, q_rot, kv.pool, kv.page_size, kv.block_tables, ctx.attn_meta,
                             self.p("sink") if self.has_sink else None, gate, o_lat, self.scale, window=self.window)
        o_heads = ctx.buffer("latent_o_heads", (H, T, V), dt)
        ops.batched_heads_mm(o_lat, self._uv_t, o_heads)
        o_rows = ctx.buffer("attn_out", (T, H * V), dt)
        ops.heads_to_rows(o_heads, o_rows)
        return self.o_proj.forward(o_rows, ctx, "mixer_out", out_dtype=self.out_dtype)


register_mixer("latent_attention", LatentAttention)
