"""A decoder model put together from a plan: embedding, blocks, final norm, head.

The plan is data.  ``blocks`` lists the layers that exist (each with its own mixer,
feed-forward and norm kinds, so layers may differ); ``schedule`` lists the order in which
they run: a ``LayerCall`` names the block, the cache slot its mixer uses and whether it
writes to it.  A block may be named twice (each call then has a cache slot of its own, or
shares one), and a call may read a slot that an earlier call wrote
(``writes_cache=False``).  The reference runs its ``ModuleList`` once in order
(models/qwen3.py:86-92); that is the schedule ``[(i, i, True) for i in range(L)]``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Iterator, Optional

import torch

from .base import Part, ParamDecl
from .block import BlockSpec, SharedRef
from .embed import LMHead, TokenEmbedding
from .registry import PartSpec, build_block, build_part


@dataclass(frozen=True)
class LayerCall:
    block: int
    cache_slot: int
    writes_cache: bool = True
    kv_slot: "Optional[int]" = None    # a mixer that reads ANOTHER call's keys and values: the cache slot that holds them
    add_row: "Optional[int]" = None    # the row of the model's pass vectors that joins the stream right before this call


@dataclass
class ModelPlan:
    vocab_size: int
    hidden_size: int
    blocks: list[BlockSpec]
    schedule: list[LayerCall]
    final_norm: PartSpec
    tie_word_embeddings: bool
    max_position: int
    shared: dict[str, PartSpec] = field(default_factory=dict)   # key -> position encoding built once
    embed_prefix: str = "model.embed_tokens."
    block_prefix: str = "model.layers.{i}."
    final_norm_prefix: str = "model.norm."
    head_prefix: str = "lm_head."
    embed_param: str = "weight"        # the tensors' names behind those prefixes
    head_param: str = "weight"
    embedding_scale: float = 1.0       # the embedding's rows are multiplied by this
    tables: dict[str, tuple[str, int, int]] = field(default_factory=dict)   # key -> (tensor name, rows, columns): tables
                                       # indexed by token that blocks share (``SharedRef(key)`` in a ``BlockSpec``'s args)
    streams: int = 1                   # residual streams; > 1: the residual is [streams, T, hidden], all equal at the start
    logit_softcap: "Optional[float]" = None   # logits <- cap * tanh(logits / cap)
    logit_scale: float = 1.0           # logits are multiplied by this (in front of the cap)
    embed_norm: "Optional[PartSpec]" = None    # a norm that the embedding passes through before it becomes the residual stream
                                       # (a norm kind with ``normalize_stream``)
    embed_norm_prefix: str = ""
    pass_vectors: "Optional[tuple[str, int]]" = None   # (tensor name, rows): vectors of ``hidden_size`` values of which a
                                       # ``LayerCall.add_row`` names one (what each pass over looped layers adds to the stream)


class PassVectors(Part):
    """Vectors [rows, width] that the model owns; a ``LayerCall`` with ``add_row`` has one of them added to the residual
    stream right before its block runs (by the block's first kernel: the block kind must set ``takes_pass_vector``)."""
    capturable = True

    def __init__(self, name: str, rows: int, width: int):
        super().__init__()
        self.name, self.rows, self.width = name, rows, width

    def param_decls(self):
        return [ParamDecl(self.name, (self.rows, self.width), role="vector")]

    def row(self, i: int) -> torch.Tensor:
        return self.p(self.name)[i]


class DecoderModel(Part):
    capturable = True

    def __init__(self, plan: ModelPlan):
        super().__init__()
        self.plan = plan
        self.shared = {k: build_part("position_encoding", s) for k, s in plan.shared.items()}
        self.embed = TokenEmbedding(plan.vocab_size, plan.hidden_size, scale=plan.embedding_scale, streams=plan.streams,
                                    param=plan.embed_param)
        self.embed_norm = build_part("norm", plan.embed_norm) if plan.embed_norm is not None else None
        if self.embed_norm is not None and not hasattr(self.embed_norm, "normalize_stream"):
            raise ValueError(f"norm kind {plan.embed_norm.kind!r} cannot normalise the stream in place (ModelPlan.embed_norm)")
        self.tables = {k: TokenEmbedding(rows, cols, param=name) for k, (name, rows, cols) in plan.tables.items()}
        self.shared.update(self.tables)
        self.pass_vectors = None
        if plan.pass_vectors is not None:
            self.pass_vectors = self.shared["pass_vectors"] = PassVectors(plan.pass_vectors[0], plan.pass_vectors[1], plan.hidden_size)
        self.blocks = [build_block(s, self.shared) for s in plan.blocks]
        self.final_norm = build_part("norm", plan.final_norm)
        tied = plan.embed_prefix + plan.embed_param if plan.tie_word_embeddings else None
        self.head = LMHead(plan.vocab_size, plan.hidden_size, tied, param=plan.head_param, softcap=plan.logit_softcap,
                           scale=plan.logit_scale)
        self.schedule = list(plan.schedule)
        n_slots = 1 + max((c.cache_slot for c in self.schedule), default=-1)
        # What each cache slot must hold, taken from the first call that uses it.
        self.slot_needs: list[list[Any]] = [[] for _ in range(n_slots)]
        written = set()
        for c in self.schedule:
            if not 0 <= c.block < len(self.blocks):
                raise ValueError(f"schedule names block {c.block}, the model has {len(self.blocks)}")
            if c.add_row is not None:
                if not getattr(self.blocks[c.block], "takes_pass_vector", False):
                    raise ValueError(f"block {c.block} ({plan.blocks[c.block].kind!r}) cannot add a pass vector in front of itself")
                if self.pass_vectors is None or not 0 <= c.add_row < self.pass_vectors.rows:
                    raise ValueError(f"the schedule names pass vector {c.add_row}, the model has "
                                     f"{self.pass_vectors.rows if self.pass_vectors else 0}")
            needs = self.blocks[c.block].cache_needs()
            if not self.slot_needs[c.cache_slot]:
                self.slot_needs[c.cache_slot] = needs
            elif self.slot_needs[c.cache_slot] != needs:
                raise ValueError(f"cache slot {c.cache_slot} is used by mixers with different needs")
            if c.writes_cache:
                written.add(c.cache_slot)
            elif c.cache_slot not in written:
                raise ValueError(f"cache slot {c.cache_slot} is read before any call writes it")
            if c.kv_slot is not None and c.kv_slot not in written:
                raise ValueError(f"cache slot {c.kv_slot} is read (kv_slot) before any call writes it")

    # ---- structure -----------------------------------------------------------------
    def sub_parts(self):
        parts = [(self.plan.embed_prefix, self.embed)]
        if self.embed_norm is not None:
            parts.append((self.plan.embed_norm_prefix, self.embed_norm))
        parts += [("", t) for t in self.tables.values()]
        if self.pass_vectors is not None:
            parts.append(("", self.pass_vectors))
        parts += [(self.plan.block_prefix.format(i=i), b) for i, b in enumerate(self.blocks)]
        parts += [(self.plan.final_norm_prefix, self.final_norm), (self.plan.head_prefix, self.head)]
        return parts

    def walk(self) -> Iterator[tuple[str, Part]]:
        """Every part once, with the prefix of its parameters (shared parts under their first owner)."""
        seen: set[int] = set()

        def rec(prefix: str, part: Part):
            if id(part) in seen:
                return
            seen.add(id(part))
            yield prefix, part
            for rel, sub in part.sub_parts():
                yield from rec(prefix + rel, sub)

        yield from rec("", self)

    def finalize_all(self, dtype, device):
        for _, part in self.walk():
            part.finalize(dtype, device)

    # ---- one step ------------------------------------------------------------------
    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        """Hidden states of the wanted rows, normalised: ``[len(ctx.logits_rows), hidden]``."""
        ctx.token_ids = token_ids
        ctx.forward_serial = getattr(ctx, "forward_serial", 0) + 1      # what parts cache for ONE pass over the layers is keyed by this
        residual = self.embed.forward(token_ids, ctx)
        delta = self.embed_norm.normalize_stream(residual, ctx) if self.embed_norm is not None else None
        for i, call in enumerate(self.schedule):
            # the block learns what runs after it, so that its last kernel can prepare for it
            after = self.blocks[self.schedule[i + 1].block].upcoming() if i + 1 < len(self.schedule) else None
            delta = self.blocks[call.block].forward(residual, delta, ctx, call, upcoming=after)
        return self.final_norm.forward(residual, delta, ctx, rows=ctx.logits_rows)

    def compute_logits(self, hidden: torch.Tensor, ctx) -> torch.Tensor:
        return self.head.forward(hidden, ctx)
