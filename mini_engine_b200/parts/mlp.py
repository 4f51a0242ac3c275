"""SwiGLU feed-forward: ``down( silu(gate(x)) * up(x) )``.

Reference: models/qwen3.py:42-51, layers/activation.py:4-7; gate and up are packed into
one weight (rows gate | up) so that one product reads x once, and SiLU-and-multiply runs in
that product's epilogue.
"""
from __future__ import annotations

from .base import FeedForward
from .linear import Linear
from .registry import register_feed_forward


class SwiGLU(FeedForward):
    capturable = True
    # In a decode step the first projection finishes the norm in front of it (the rows' factors applied to its
    # results) and the last one adds into the residual stream and starts the next norm, all in their epilogues.
    takes_pending_norm = True
    adds_to_residual = True

    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__()
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.gate_up_proj = Linear(hidden_size, [("gate_proj.weight", intermediate_size),
                                                 ("up_proj.weight", intermediate_size)],
                                   name="gate_up_proj.weight")
        self.down_proj = Linear(intermediate_size, [("down_proj.weight", hidden_size)],
                                name="down_proj.weight")

    def sub_parts(self):
        return [("", self.gate_up_proj), ("", self.down_proj)]

    def first_weight(self):
        return self.gate_up_proj.weight

    def forward(self, x, ctx, residual=None, upcoming=None):
        act = self.gate_up_proj.forward(x, ctx, "ffn_act", epilogue="silu_mul", fetch_ahead=self.down_proj.weight)
        return self.down_proj.forward(act, ctx, "ffn_out", may_split=True, residual=residual,
                                      next_norm=upcoming.norm if upcoming else None,
                                      fetch_ahead=upcoming.weight if upcoming else None)


class ActivationMLP(FeedForward):
    """``down(act(up(x)))`` with an element-wise activation (a key of ``ops.ACTIVATIONS``; "relu_squared" is max(z, 0)^2)."""
    capturable = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu_squared", up: str = "up", down: str = "down"):
        super().__init__()
        from .. import ops
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(ops.ACTIVATIONS)}")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.up = Linear(hidden_size, [(up, intermediate_size)], name=up)
        self.down = Linear(intermediate_size, [(down, hidden_size)], name=down)

    def sub_parts(self):
        return [("", self.up), ("", self.down)]

    def first_weight(self):
        return self.up.weight

    def forward(self, x, ctx, out_name: str = "ffn_out"):
        from .. import ops
        z = self.up.forward(x, ctx, out_name + "_up", epilogue=self.activation if self.up.fuses(x, ctx, self.activation) else "none")
        if not self.up.fuses(x, ctx, self.activation):
            act = ctx.buffer(out_name + "_act", tuple(z.shape), ctx.act_dtype)
            ops.activation(z, act, self.activation)
            z = act
        return self.down.forward(z, ctx, out_name)


register_feed_forward("swiglu", SwiGLU)
register_feed_forward("activation_mlp", ActivationMLP)
