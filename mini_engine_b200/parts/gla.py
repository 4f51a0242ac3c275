"""Gated linear attention as a mixer with a state slot per request.

Per head: q = W_q h * dim^-1/2, k = W_k h (``dim`` values), v = W_v h (``vdim`` values) and a decay per key channel
a = sigmoid(z)^(1/tau) with z = W_a2 (W_a1 h) + b (a low-rank projection); then

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,        o_t = S_t^T q_t          (S starts at zero)

Every head's o is brought to unit root mean square and scaled by one weight vector of ``vdim`` values (the same for all
heads); the joined heads then pass the gate silu(W_g h) and the output product W_o.  S is float32 and lives in the request's state
slot; decays, their logarithms and everything of the recurrence are float32 (the packed projection returns float32).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, ParamDecl, StateNeed
from .linear import Linear
from .registry import register_mixer


class GatedLinearAttention(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, decay_rank: int, tau: float, norm_eps: float):
        super().__init__()
        if not tau > 0:
            raise ValueError(f"tau must be positive, got {tau}")
        if min(num_heads, dim, vdim, decay_rank) < 1:
            raise ValueError("GatedLinearAttention: sizes must be positive")
        self.hidden_size, self.num_heads, self.dim, self.vdim = hidden_size, num_heads, dim, vdim
        self.decay_rank, self.tau, self.norm_eps = decay_rank, float(tau), float(norm_eps)
        H = num_heads
        pieces = [("q", H * dim), ("k", H * dim), ("v", H * vdim), ("g", H * vdim), ("a1", decay_rank)]
        self.in_proj = Linear(hidden_size, pieces, name="in_proj")
        self.offsets, off = {}, 0
        for name, rows in pieces:
            self.offsets[name] = off
            off += rows
        self.o_proj = Linear(H * vdim, [("o", hidden_size)], name="o")

    def sub_parts(self):
        return [("", self.in_proj), ("", self.o_proj)]

    def param_decls(self):
        C = self.num_heads * self.dim
        return [ParamDecl("a2", (C, self.decay_rank)), ParamDecl("a2.b", (C,), role="vector"),
                ParamDecl("norm", (self.vdim,), init="norm", role="vector")]

    def cache_needs(self):
        return [StateNeed((self.num_heads, self.dim, self.vdim), "float32", "S")]

    def first_weight(self):
        return self.in_proj.weight

    def forward(self, x, ctx, call):
        H, D, V = self.num_heads, self.dim, self.vdim
        proj = self.in_proj.forward(x, ctx, "gla_proj", out_dtype=torch.float32)
        T = proj.shape[0]
        la = ctx.buffer("gla_log_decay", (T, H * D), torch.float32)
        ops.gla_decay(proj, self.offsets["a1"], self.decay_rank, self.p("a2"), self.p("a2.b"), self.tau, la)
        o = ctx.buffer("gla_o", (T, H * V), torch.float32)
        runs = ops.gla_chunk_count(ctx.attn_meta)
        scores = ctx.buffer("gla_scores", (T, H, ops.GLA_CHUNK), torch.float32) if runs else None
        chunk_states = ctx.buffer("gla_chunk_states", (runs, H, D, V), torch.float32) if runs else None
        ops.gla_scan(proj, self.offsets, la, ctx.state(call.cache_slot, "S"), ctx.attn_meta, ctx.state_slots, o, H, D, V, D ** -0.5,
                     scores=scores, chunk_states=chunk_states)
        gated = ctx.buffer("gla_gated", (T, H * V), ctx.act_dtype)
        ops.mlstm_out(o, proj, self.offsets["g"], self.p("norm"), self.norm_eps, gated, H, V, shared_weight=True, gate="silu")
        return self.o_proj.forward(gated, ctx, "mixer_out")


register_mixer("gla", GatedLinearAttention)
