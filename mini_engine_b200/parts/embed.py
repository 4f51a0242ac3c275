"""Token embedding and output head.

Reference: layers/embed_head.py:5-23.  The embedding writes the float32 residual stream;
the head takes the rows that were asked for (already gathered and normalised) and returns
float32 logits.  A tied head shares the embedding's storage (models/qwen3.py:107-109).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import ParamDecl, Part


class TokenEmbedding(Part):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, streams: int = 1, param: str = "weight"):
        super().__init__()
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.scale = float(scale)          # rows are multiplied by this
        self.streams = streams             # > 1: the residual is [streams, T, hidden], every stream the embedding
        self.param = param

    def param_decls(self):
        return [ParamDecl(self.param, (self.vocab_size, self.hidden_size))]

    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        shape = (token_ids.shape[0], self.hidden_size)
        out = ctx.buffer("residual", shape if self.streams == 1 else (self.streams, *shape), torch.float32)
        ops.embed(token_ids, self.p(self.param), out, ctx.error_flag, feedback=getattr(ctx, "token_feedback", None),
                  scale=self.scale)
        return out


class LMHead(Part):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: str | None, param: str = "weight", softcap: float | None = None,
                 scale: float = 1.0):
        super().__init__()
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied_to = tied_to
        self.param = param
        self.softcap = float(softcap) if softcap else None     # logits <- cap * tanh(logits / cap)
        self.scale = float(scale)                              # ... of the logits times this

    def param_decls(self):
        return [ParamDecl(self.param, (self.vocab_size, self.hidden_size), tied_to=self.tied_to)]

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        out = ctx.buffer("logits", (x.shape[0], self.vocab_size), torch.float32)
        ops.tag = "logits"
        ops.linear(x, self.p(self.param), out, workspace=ctx.buffer, err=ctx.error_flag)
        if self.softcap or self.scale != 1.0:
            ops.soft_cap(out, self.softcap, self.scale)
        return out
