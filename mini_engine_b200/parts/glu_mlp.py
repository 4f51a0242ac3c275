"""Gated feed-forwards whose two halves are clamped, dense or as a mixture of routed experts.

One expert (and the dense form): g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit),
y = g * sigmoid(alpha * g) * (u + shift), output W_down y; ``limit`` None: nothing is clamped.  ``alpha`` 1 and ``shift`` 0
is the plain SiLU-gated form silu(g) * u.

``RoutedExperts``: router logits z = W_router h + b in float32; a token goes to its ``top`` experts of largest
logit, mixed by a softmax taken over those ``top`` logits alone; the output is that mix of their outputs, plus a
``shared`` expert (same form, sizes of its own) that runs for every token.  Routing, grouping by expert, the per-expert
products and the weighted sum all run on the device, so a step's shape does not depend on the routing.

Two more choices.  ``routing`` "sigmoid_groups" (instead of "softmax_top"): scores s = sigmoid(z); the choice is made by
s + ``correction`` (a learned number per expert that only steers the choice); the experts form ``groups`` = (count, keep)
equal groups of neighbours, a group's score is the sum of its two largest choice scores, and only experts of the ``keep``
best groups can be chosen; the weights are the chosen experts' s, not renormalised.  ``activation`` (a key of
``ops.ACTIVATIONS``, instead of the gate): an expert is W_down act(W_up h) and has no gate matrix.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import DiskSource, FeedForward, ParamDecl
from .linear import Linear
from .registry import register_feed_forward


class ClampedGLU(FeedForward):
    capturable = True

    def __init__(self, hidden_size: int, intermediate_size: int, limit: Optional[float] = None, alpha: float = 1.702,
                 shift: float = 1.0, gate: str = "gate", up: str = "up", down: str = "down"):
        super().__init__()
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.limit = float(limit) if limit is not None else 0.0
        self.alpha = float(alpha)
        self.shift = float(shift)
        self.gate_up = Linear(hidden_size, [(gate, intermediate_size), (up, intermediate_size)], name="gate_up")
        self.down = Linear(intermediate_size, [(down, hidden_size)], name=down)

    def sub_parts(self):
        return [("", self.gate_up), ("", self.down)]

    def first_weight(self):
        return self.gate_up.weight

    def forward(self, x, ctx, out_name: str = "ffn_out", out_dtype=None):
        act = ctx.buffer(out_name + "_act", (x.shape[0], self.intermediate_size), ctx.act_dtype)
        w = self.gate_up.weight
        if (ctx.act_dtype == torch.bfloat16 and ops.use_tcgen05_gemm and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and ops.tcgen05_takes(x, w)):
            # a long step: the activation is the epilogue of the tcgen05 product, as SiLU is in a SwiGLU
            ops.tag = out_name + "_act"
            ops.linear_tcgen05(x, w, act, "silu_mul", ctx.error_flag, glu=(self.limit, self.alpha, self.shift))
        elif (ctx.act_dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
              and ops.decode_linear_takes(x.shape[0], self.hidden_size, w, False)):
            # a step of up to 16 tokens: the same in the epilogue of the decode products
            ops.tag = out_name + "_act"
            ops.decode_linear(w, x, out=act, epilogue="silu_mul", fetch_ahead=self.down.weight, err=ctx.error_flag,
                              glu=(self.limit, self.alpha, self.shift))
        else:
            z = self.gate_up.forward(x, ctx, out_name + "_gate_up")
            ops.clamped_glu(z, act, self.limit, self.alpha, self.shift)
        return self.down.forward(act, ctx, out_name, out_dtype=out_dtype)


class RoutedExperts(FeedForward):
    capturable = True

    def __init__(self, hidden_size: int, num_experts: int, top: int, expert_size: int, limit: Optional[float] = None,
                 alpha: float = 1.702, shift: float = 1.0, router_bias: bool = True, shared: Optional[dict] = None,
                 routing: str = "softmax_top", groups: Optional[tuple] = None, correction: bool = False,
                 activation: Optional[str] = None, out_dtype: Optional[str] = None):
        super().__init__()
        if not 1 <= top <= num_experts:
            raise ValueError(f"{top} of {num_experts} experts cannot be chosen")
        if routing not in ("softmax_top", "sigmoid_groups"):
            raise ValueError(f"routing must be 'softmax_top' or 'sigmoid_groups', got {routing!r}")
        if activation is not None and activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(ops.ACTIVATIONS)}")
        count, keep = (int(groups[0]), int(groups[1])) if groups else (1, 1)
        if routing == "sigmoid_groups" and (count < 1 or num_experts % count or not 1 <= keep <= count
                                            or keep * (num_experts // count) < top):
            raise ValueError(f"{keep} of {count} groups over {num_experts} experts cannot give {top} choices")
        if routing == "softmax_top" and (groups or correction):
            raise ValueError("groups and a correction go with routing 'sigmoid_groups'")
        self.routing, self.groups, self.has_correction, self.activation = routing, (count, keep), correction, activation
        self.out_dtype = getattr(torch, out_dtype) if out_dtype else None    # what the weighted sum is written as (None: the working dtype)
        self.hidden_size, self.num_experts, self.top, self.expert_size = hidden_size, num_experts, top, expert_size
        self.limit = float(limit) if limit is not None else 0.0
        self.alpha = float(alpha)
        self.shift = float(shift)
        self.has_router_bias = router_bias and routing == "softmax_top"
        self.router = Linear(hidden_size, [("router", num_experts)], name="router")
        self.shared = ClampedGLU(hidden_size, **shared) if shared else None
        self._gate_up = self._down = None

    def sub_parts(self):
        return [("", self.router)] + ([("shared.", self.shared)] if self.shared is not None else [])

    def param_decls(self):
        E, F, W = self.num_experts, self.expert_size, self.hidden_size
        gate_up, down = [], []
        rows = F if self.activation else 2 * F          # an expert's rows in the first packed matrix: up, or gate then up
        for e in range(E):
            if self.activation:
                gate_up.append(DiskSource(f"e{e}.up", F * e, F))
            else:
                gate_up += [DiskSource(f"e{e}.gate", 2 * F * e, F), DiskSource(f"e{e}.up", 2 * F * e + F, F)]
            down.append(DiskSource(f"e{e}.down", W * e, W))
        decls = [ParamDecl("experts_gate_up", (E * rows, W), sources=gate_up), ParamDecl("experts_down", (E * W, F), sources=down)]
        if self.has_router_bias:
            decls.append(ParamDecl("router.b", (E,), role="vector"))
        if self.has_correction:
            decls.append(ParamDecl("correction", (E,), role="vector"))
        return decls

    def first_weight(self):
        return self.router.weight

    def finalize(self, dtype, device):
        E, F, W = self.num_experts, self.expert_size, self.hidden_size
        self._gate_up = self.p("experts_gate_up").view(E, F if self.activation else 2 * F, W)
        self._down = self.p("experts_down").view(E, W, F)

    def forward(self, x, ctx):
        E, F, W, top = self.num_experts, self.expert_size, self.hidden_size, self.top
        T = x.shape[0]
        z = self.router.forward(x, ctx, "moe_logits", out_dtype=torch.float32)
        idx = ctx.buffer("moe_idx", (T, top), torch.int32)
        wgt = ctx.buffer("moe_weights", (T, top), torch.float32)
        counts = ctx.buffer("moe_counts", (E,), torch.int32)
        offsets = ctx.buffer("moe_offsets", (E + 1,), torch.int32)
        order = ctx.buffer("moe_order", (T * top,), torch.int32)
        place = ctx.buffer("moe_place", (T * top,), torch.int32)
        if self.routing == "sigmoid_groups":
            ops.moe_route_grouped_sort(z, self.p("correction") if self.has_correction else None, top, *self.groups, idx, wgt, counts,
                                       offsets, order, place)
        else:
            ops.moe_route_sort(z, self.p("router.b") if self.has_router_bias else None, top, idx, wgt, counts, offsets, order, place)
        act = ctx.buffer("moe_act", (T * top, F), ctx.act_dtype)
        if self.activation:
            ops.moe_gemm(x, order, top, self._gate_up, offsets, act, activation=self.activation, workspace=ctx.buffer, err=ctx.error_flag)
        else:
            ops.moe_gemm(x, order, top, self._gate_up, offsets, act, glu=(self.limit, self.alpha, self.shift), workspace=ctx.buffer,
                         err=ctx.error_flag)
        rows = ctx.buffer("moe_rows", (T * top, W), torch.float32)
        ops.moe_gemm(act, None, top, self._down, offsets, rows, workspace=ctx.buffer, err=ctx.error_flag)
        shared = self.shared.forward(x, ctx, out_name="moe_shared") if self.shared is not None else None
        out = ctx.buffer("ffn_out", (T, W), self.out_dtype or ctx.act_dtype)
        ops.moe_combine(rows, place, wgt, shared, out)
        return out


register_feed_forward("clamped_glu", ClampedGLU)
register_feed_forward("routed_experts", RoutedExperts)
