"""One decoder block: how norm, mixer and feed-forward are arranged around the residual.

Reference wiring (models/qwen3.py:65-74, layers/layernorm.py:19-23): pre-norm, with each
sub-layer's output added to the residual inside the next norm.  The same deferred add is
used here: a block receives the residual stream and the previous sub-layer's output
(``delta``, not yet added) and returns its own last output the same way.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from .base import NormedUpdate, ParamDecl, Part, PendingSum, StreamCopy, StreamUpdate, Upcoming
from .registry import PartSpec, build_part, register_block


@dataclass
class BlockSpec:
    """One layer as data: the parts it is made of and (``kind``) how they are arranged.

    ``norm`` is the norm of both places; ``mixer_norm`` / ``feed_forward_norm`` give a place a norm of its own."""
    mixer: PartSpec
    feed_forward: Optional[PartSpec]   # None: a layer without a feed-forward (for block kinds that allow it)
    norm: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    kind: str = "pre_norm"             # a name registered with ``register_block``
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    feed_forward_norm_prefix: str = "post_attention_layernorm."
    args: dict[str, Any] = field(default_factory=dict)   # what the block kind itself needs (streams, taps, ...)

    def norm_of(self, place: str) -> PartSpec:
        spec = getattr(self, place) or self.norm
        if spec is None:
            raise ValueError(f"a block needs a norm for {place!r} (give ``norm`` or ``{place}``)")
        return spec


class Block(Part):
    """The arrangement of a layer's parts around the residual stream; built by the factory registered for
    ``BlockSpec.kind``.

    What the model asks of a block: ``mixer`` (its ``cache_needs()`` decide the layer's cache slot),
    ``sub_parts()`` (for the weights), ``upcoming()`` (what the block starts with, for the block before it; may be
    an empty ``Upcoming``) and ``forward(residual, delta, ctx, call, upcoming=None)``: ``residual`` is the float32
    stream [T, hidden], updated in place; ``delta`` is the output of the block before that is not added yet (a
    tensor, float32 split-K partial results, ``AddedToResidual``, or None); the return value is this block's own
    last output in the same form (None: everything is in ``residual`` already)."""

    mixer: Part

    def __init__(self, spec: BlockSpec, shared: Optional[dict] = None):
        super().__init__()
        self.spec = spec
        mixer_spec = spec.mixer
        if shared:
            # Objects that several layers share (one rotary table for all of them).
            args = {k: shared.get(v.key, v) if isinstance(v, SharedRef) else v
                    for k, v in mixer_spec.args.items()}
            mixer_spec = PartSpec(mixer_spec.kind, args)
        self.mixer = build_part("mixer", mixer_spec)
        self.mixer_norm = build_part("norm", spec.norm_of("mixer_norm"))
        self.feed_forward = self.feed_forward_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = build_part("feed_forward", spec.feed_forward)
            self.feed_forward_norm = build_part("norm", spec.norm_of("feed_forward_norm"))
        elif not self.feed_forward_optional:
            raise ValueError(f"a {spec.kind!r} block needs a feed-forward")

    feed_forward_optional = False

    def sub_parts(self):
        s = self.spec
        parts = [(s.mixer_norm_prefix, self.mixer_norm), (s.mixer_prefix, self.mixer)]
        if self.feed_forward is not None:
            parts += [(s.feed_forward_norm_prefix, self.feed_forward_norm), (s.feed_forward_prefix, self.feed_forward)]
        return parts

    def cache_needs(self):
        """What one call of this block needs of the cache: the mixer's needs, and the block's own if it has any."""
        return self.mixer.cache_needs()

    def upcoming(self) -> Upcoming:
        return Upcoming()

    def forward(self, residual, delta, ctx, call, upcoming=None):
        raise NotImplementedError


class PreNormBlock(Block):
    """``r += mixer(norm(r)); r += feed_forward(norm(r))`` with each sum deferred into the norm that follows
    (models/qwen3.py:65-74 in the reference)."""
    capturable = True

    def upcoming(self) -> Upcoming:
        """What this block starts with, for the block that runs before it."""
        return Upcoming(self.mixer_norm, self.mixer.first_weight())

    def forward(self, residual, delta, ctx, call, upcoming=None):
        """``delta``: the output of the sub-layer before this block, not yet added to ``residual`` (or the mark
        that it has been).  Returns this block's last output the same way.  ``upcoming``: what runs after this
        block (``Upcoming``), if the caller knows it."""
        mixer, ffn = self.mixer, self.feed_forward
        x = self.mixer_norm.forward(residual, delta, ctx, lazy=mixer.takes_pending_norm)
        if mixer.adds_to_residual:
            mixed = mixer.forward(x, ctx, call, residual=residual,
                                  upcoming=Upcoming(self.feed_forward_norm, ffn.first_weight()))
        else:
            mixed = mixer.forward(x, ctx, call)
        x = self.feed_forward_norm.forward(residual, mixed, ctx, lazy=ffn.takes_pending_norm)
        if ffn.adds_to_residual:
            return ffn.forward(x, ctx, residual=residual, upcoming=upcoming)
        return ffn.forward(x, ctx)


class HyperConnectionBlock(Block):
    """A pre-norm block over several residual streams, with a short convolution in front of each sub-layer.

    The model keeps ``streams`` copies x_1 .. x_S of the residual stream ([S, T, width] float32).  Sub-layer q (1: mixer,
    2: feed-forward) reads u = sum_s in_q[s] x_s, computes y = sublayer(h + conv_q(h)) with h = norm_q(u) and
    conv_q a causal convolution of ``taps`` taps over time on each channel, and all streams are renewed at once:
    x_r <- sum_s mix_q[s, r] x_s + out_q[r] y.  That last step is left to the kernel that reads the streams next (the
    following norm), so a block returns its last y as a ``StreamUpdate``.  The block's own parameters are
    ``hc1.in / hc1.out / hc1.mix`` (and ``hc2.*``) and the convolutions ``canon1`` / ``canon2``, whose last inputs are
    part of a request's state.  The feed-forward may be absent.

    ``BlockSpec.args``: ``streams``, ``width``, ``taps``."""
    capturable = True
    feed_forward_optional = True

    def __init__(self, spec: BlockSpec, shared: Optional[dict] = None):
        super().__init__(spec, shared)
        from .conv import CausalShortConv
        self.streams = int(spec.args["streams"])
        self.width = int(spec.args["width"])
        taps = int(spec.args["taps"])
        self.conv1 = CausalShortConv(self.width, taps, param="canon1", state_name="canon1")
        self.conv2 = CausalShortConv(self.width, taps, param="canon2", state_name="canon2") if self.feed_forward is not None else None

    def sub_parts(self):
        parts = super().sub_parts() + [("", self.conv1)]
        if self.conv2 is not None:
            parts.append(("", self.conv2))
        return parts

    def param_decls(self):
        S = self.streams
        decls = []
        for q in ("hc1", "hc2") if self.feed_forward is not None else ("hc1",):
            decls += [ParamDecl(q + ".in", (S,), init="norm", role="vector"), ParamDecl(q + ".out", (S,), init="norm", role="vector"),
                      ParamDecl(q + ".mix", (S, S), init="eye", role="vector")]
        return decls

    def cache_needs(self):
        needs = self.mixer.cache_needs() + self.conv1.cache_needs()
        return needs + (self.conv2.cache_needs() if self.conv2 is not None else [])

    def forward(self, residual, delta, ctx, call, upcoming=None):
        """``residual`` [streams, T, width]; ``delta``: the ``StreamUpdate`` the block before left (or None)."""
        y = self.mixer.forward(self._normed(self.mixer_norm, self.conv1, "hc1.in", residual, delta, ctx, call), ctx, call)
        update = StreamUpdate(y, self.p("hc1.mix"), self.p("hc1.out"))
        if self.feed_forward is None:
            return update
        y = self.feed_forward.forward(self._normed(self.feed_forward_norm, self.conv2, "hc2.in", residual, update, ctx, call), ctx)
        return StreamUpdate(y, self.p("hc2.mix"), self.p("hc2.out"))

    def _normed(self, norm, conv, mix_in, residual, delta, ctx, call):
        """What a sub-layer reads: the pending update, the mix of the streams, the norm and h + conv(h).  In a step where
        every request brings one token the convolution needs no neighbour and runs inside the norm's kernel."""
        import torch
        meta = ctx.attn_meta
        if self.fuse_decode_conv and meta.num_decodes == meta.num_reqs and conv.residual and hasattr(norm, "param"):
            state = ctx.state(call.cache_slot, conv.state_name) if conv.taps > 1 else None
            return norm.forward(residual, delta, ctx, mix_in=self.p(mix_in), out_name="conv_out", conv=(conv.p(conv.param), state))
        h = norm.forward(residual, delta, ctx, mix_in=self.p(mix_in), out_dtype=torch.float32, out_name="norm_h")
        return conv.forward(h, ctx, call.cache_slot)

    fuse_decode_conv = True      # a switch for comparisons


class SandwichNormBlock(Block):
    """A block whose sub-layers are normalised on both sides: x <- x + mult * norm_b(sublayer(norm_a(x))) for the mixer
    and then for the feed-forward (which may be absent), and after them, optionally, a per-layer input from the token
    itself: x <- x + mult * rms_norm(side(x)) with a plain weight.  Each of these sums is left pending (``NormedUpdate``)
    and done by the kernel that reads the stream next: the following norm, or the copy of the stream that the token
    input reads.

    ``BlockSpec.args``: ``mult``; ``width``; ``post_mixer_norm`` / ``post_feed_forward_norm`` (the ``PartSpec`` of the norm
    behind each sub-layer); ``side`` = {dim, first, table: SharedRef} or absent."""
    capturable = True
    feed_forward_optional = True

    def __init__(self, spec: BlockSpec, shared: Optional[dict] = None):
        super().__init__(spec, shared)
        from .token_side import TokenSideInput
        a = spec.args
        self.mult = float(a.get("mult", 1.0))
        self.post_mixer_norm = build_part("norm", a["post_mixer_norm"])
        self.post_feed_forward_norm = build_part("norm", a["post_feed_forward_norm"]) if self.feed_forward is not None else None
        self.side = None
        if a.get("side"):
            side = a["side"]
            table = (shared or {}).get(side["table"].key) if isinstance(side["table"], SharedRef) else side["table"]
            if table is None:
                raise ValueError("a block's token input needs the model's table (ModelPlan.tables)")
            self.side = TokenSideInput(a["width"], side["dim"], side["first"], table)

    def sub_parts(self):
        parts = super().sub_parts() + [("", self.post_mixer_norm)]
        if self.post_feed_forward_norm is not None:
            parts.append(("", self.post_feed_forward_norm))
        if self.side is not None:
            parts.append(("", self.side))
        return parts

    def upcoming(self) -> Upcoming:
        return Upcoming(self.mixer_norm, self.mixer.first_weight())

    def forward(self, residual, delta, ctx, call, upcoming=None):
        from .. import ops
        eps = self.mixer_norm.eps
        y = self.mixer.forward(self.mixer_norm.forward(residual, delta, ctx), ctx, call)
        update = NormedUpdate(y, self.post_mixer_norm.weight, eps, self.mult)
        if self.feed_forward is not None:
            y = self.feed_forward.forward(self.feed_forward_norm.forward(residual, update, ctx), ctx)
            update = NormedUpdate(y, self.post_feed_forward_norm.weight, eps, self.mult)
        if self.side is not None:
            x = ctx.buffer("stream_copy", tuple(residual.shape), ctx.act_dtype)
            ops.sandwich_norm(residual, update.y, update.weight, update.mult, None, eps, x, norm_out=False)
            update = NormedUpdate(self.side.forward(x, ctx), self.side.p(self.side.norm), eps, self.mult)
        return update


class ParallelBlock(Block):
    """A block whose mixer and feed-forward read the same residual stream, each through a norm of its own:
    x <- x + (mixer(norm1(x)) + feed_forward(norm2(x))); the feed-forward may be absent.  Both outputs are left pending
    (``PendingSum``) and join the stream in the kernel that reads it next, which also computes both norms of the new rows in
    one pass; a mixer's output bias (``output_bias()``) is deferred the same way.  A ``LayerCall`` may name a pass vector
    (``add_row``) that joins the stream right before the block's norms.  The norms must be of a kind that takes a
    ``PendingSum`` (a layer norm with a bias)."""
    capturable = True
    feed_forward_optional = True
    takes_pass_vector = True

    def __init__(self, spec: BlockSpec, shared: Optional[dict] = None):
        super().__init__(spec, shared)
        self.pass_vectors = (shared or {}).get("pass_vectors")
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "_sum_and_norm"):
                raise ValueError("a 'parallel' block needs norms that can add a pending sum (kind 'layernorm')")
        if hasattr(self.mixer, "defer_output_bias"):
            self.mixer.defer_output_bias = True

    def param_decls(self):
        """A layer without a feed-forward has no use for the second norm; files that hold one all the same are accepted."""
        if self.feed_forward is not None:
            return []
        spec = self.spec.feed_forward_norm or self.spec.norm
        if spec is None or "size" not in spec.args:
            return []
        names = [spec.args.get("param", "weight")] + ([spec.args["bias"]] if spec.args.get("bias") else [])
        return [ParamDecl(self.spec.feed_forward_norm_prefix + n, (spec.args["size"],), role="vector", optional=True) for n in names]

    def forward(self, residual, delta, ctx, call, upcoming=None):
        vectors = []
        if call.add_row is not None:
            vectors.append(self.pass_vectors.row(call.add_row))
        also = (self.feed_forward_norm, "norm_out2") if self.feed_forward is not None else None
        h = self.mixer_norm._sum_and_norm(residual, delta, ctx, None, "norm_out", None, vectors=vectors, also=also)
        h1, h2 = h if also is not None else (h, None)
        pending = PendingSum([self.mixer.forward(h1, ctx, call)])
        bias = self.mixer.output_bias() if hasattr(self.mixer, "output_bias") else None
        if bias is not None:
            pending.vectors.append(bias)
        if self.feed_forward is not None:
            pending.outputs.append(self.feed_forward.forward(h2, ctx))
        return pending


class PostNormBlock(Block):
    """A block whose norms sit behind the sub-layers and nowhere else: x <- x + norm1(mixer(x)), then x <- x + norm2(ff(x));
    the sub-layers read the stream itself, and the feed-forward may be absent.  Nothing is left pending: the norm's kernel adds
    the normalised output into the float32 stream and hands the new stream on in the working dtype (``StreamCopy``), to the
    next sub-layer and to the next block.  The norms must be of a kind with ``add_normed`` (``group_rmsnorm``)."""
    capturable = True
    feed_forward_optional = True

    def __init__(self, spec: BlockSpec, shared: Optional[dict] = None):
        super().__init__(spec, shared)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError("a 'post_norm' block needs norms that can add a normalised output to the stream (kind 'group_rmsnorm')")

    def param_decls(self):
        """A layer without a feed-forward has no use for the second norm; files that hold one all the same are accepted."""
        if self.feed_forward is not None:
            return []
        spec = self.spec.feed_forward_norm or self.spec.norm
        if spec is None or "size" not in spec.args:
            return []
        return [ParamDecl(self.spec.feed_forward_norm_prefix + spec.args.get("param", "weight"), (spec.args["size"],), role="vector",
                          optional=True)]

    def forward(self, residual, delta, ctx, call, upcoming=None):
        if isinstance(delta, StreamCopy):
            x = delta.x
        elif delta is None:
            x = residual if ctx.act_dtype == residual.dtype else residual.to(ctx.act_dtype)
        else:
            raise TypeError(f"a 'post_norm' block cannot take a pending {type(delta).__name__} from the block before it")
        update = self.mixer_norm.add_normed(residual, self.mixer.forward(x, ctx, call), ctx)
        if self.feed_forward is not None:
            update = self.feed_forward_norm.add_normed(residual, self.feed_forward.forward(update.x, ctx), ctx)
        return update


@dataclass(frozen=True)
class SharedRef:
    """Stands in a PartSpec's args for an object that the model builds once and shares."""
    key: str


register_block("pre_norm", PreNormBlock)
register_block("hyper_connection", HyperConnectionBlock)
register_block("sandwich_norm", SandwichNormBlock)
register_block("parallel", ParallelBlock)
register_block("post_norm", PostNormBlock)
