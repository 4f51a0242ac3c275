"""RMSNorm with the residual sum folded in.

Reference formula (layers/layernorm.py:11-23): ``y = x * rsqrt(mean(x^2) + eps)`` in
float32, cast to the working dtype, times the weight; with a residual the sum
``x + residual`` is normalised and also returned.  Here the residual stream itself is
kept in float32 in both precisions, so the sum, the statistics and the weight multiply
all happen in float32 and the result is rounded once.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import AddedToResidual, Norm, NormedUpdate, ParamDecl, PendingNorm, PendingSum, StreamCopy, StreamUpdate
from .registry import register_norm


class RMSNorm(Norm):
    """``param``: the weight's name on disk, for models that do not call it ``weight``.  ``unit_offset``: the weight is
    stored as its distance from one (y = x / rms(x) * (1 + w)); the sum is formed once, in float32, when the weights
    are in place.  A pending ``NormedUpdate`` (a sub-layer's output that is itself normalised, weighted and scaled before
    it joins the stream) goes into the residual in the same pass."""
    capturable = True

    def __init__(self, size: int, eps: float, param: str = "weight", unit_offset: bool = False):
        super().__init__()
        self.size = size
        self.eps = float(eps)
        self.param = param
        self.unit_offset = unit_offset
        self._weight = None

    def param_decls(self):
        return [ParamDecl(self.param, (self.size,), init="normal" if self.unit_offset else "norm", role="vector")]

    def finalize(self, dtype, device):
        self._weight = (1.0 + self.p(self.param)).contiguous() if self.unit_offset else self.p(self.param)

    @property
    def weight(self) -> torch.Tensor:
        """The factor that multiplies the normalised rows (float32)."""
        return self._weight if self._weight is not None else self.p(self.param)

    def separable_weight(self):
        """y = x * rsqrt(mean(x^2) + eps) * w splits into an element-wise x * w and one factor per row, so the part
        in front may write x * w itself."""
        return self.weight

    def forward(self, residual, delta, ctx, rows: Optional[torch.Tensor] = None, lazy: bool = False):
        n = residual.shape[0] if rows is None else rows.shape[0]
        if isinstance(delta, NormedUpdate):
            out = ctx.buffer("norm_out", (n, self.size), ctx.act_dtype)
            ops.sandwich_norm(residual, delta.y, delta.weight, delta.mult, self.weight, self.eps, out, rows=rows)
            return out
        if isinstance(delta, AddedToResidual):
            if lazy and rows is None and delta.preweighted is not None and delta.weight is self.weight:
                return PendingNorm(residual, self.weight, self.eps, delta.sumsq, delta.preweighted)
            delta = None                          # the residual already holds the sum
        out = ctx.buffer("norm_out", (n, self.size), ctx.act_dtype)
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows=rows)
        return out


class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * w`` with var the mean squared deviation, a weight and no bias, over one
    residual stream or several: with ``streams`` > 1 the residual is [streams, T, size] and the norm reads
    u = sum_s mix_in[s] x_s (every stream once when no ``mix_in`` is given: the sum of the streams).  A pending
    ``StreamUpdate`` (or, with one stream, a plain output still to be added) goes into the streams in the same pass.
    ``param``: the weight's name on disk, for models that do not call it ``weight``.  ``bias``: the name of a bias that is
    added behind the weight (one stream only); such a norm also takes a pending ``PendingSum`` (several outputs and vectors
    still to be added) and may be computed together with a second norm of the same rows (``also=(norm, out_name)``: a
    block whose sub-layers both read the stream)."""
    capturable = True

    def __init__(self, size: int, eps: float, streams: int = 1, param: str = "weight", bias: Optional[str] = None):
        super().__init__()
        if bias is not None and streams != 1:
            raise ValueError("LayerNorm: a bias is supported over one residual stream only")
        self.size = size
        self.eps = float(eps)
        self.streams = streams
        self.param = param
        self.bias = bias
        self._ones = None

    def param_decls(self):
        decls = [ParamDecl(self.param, (self.size,), init="norm", role="vector")]
        if self.bias is not None:
            decls.append(ParamDecl(self.bias, (self.size,), role="vector"))
        return decls

    def weight_and_bias(self):
        return self.p(self.param), (self.p(self.bias) if self.bias is not None else None)

    def _sum_and_norm(self, residual, delta, ctx, rows, out_name, out_dtype, vectors=(), also=None):
        """One pass of ``parallel_norm``: everything pending joins the stream, then this norm (and ``also``'s)."""
        outputs, vectors = [], list(vectors)
        if isinstance(delta, PendingSum):
            outputs, vectors = list(delta.outputs), list(delta.vectors) + vectors
        elif isinstance(delta, torch.Tensor):
            outputs = [delta]
        elif delta is not None and not isinstance(delta, AddedToResidual):
            raise TypeError(f"LayerNorm with a bias cannot add a pending {type(delta).__name__}")
        n = residual.shape[0] if rows is None else rows.shape[0]
        dtype = out_dtype or ctx.act_dtype
        out = ctx.buffer(out_name, (n, self.size), dtype)
        out2 = ctx.buffer(also[1], (n, self.size), dtype) if also is not None else None
        ops.parallel_norm(residual, outputs, vectors, self.eps, self.weight_and_bias(), out,
                          also[0].weight_and_bias() if also is not None else None, out2, rows=rows)
        return out if also is None else (out, out2)

    def forward(self, residual, delta, ctx, rows: Optional[torch.Tensor] = None, lazy: bool = False, *,
                mix_in: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None, out_name: str = "norm_out",
                conv=None):
        """``conv`` = (weight, state or None): in a step where every request brings one token, the short convolution that
        follows the norm (h + conv(h), its state moved on) runs in the norm's kernel; the result is then that sum."""
        if residual.dim() == 2 and mix_in is None and conv is None and (self.bias is not None or isinstance(delta, PendingSum)):
            return self._sum_and_norm(residual, delta, ctx, rows, out_name, out_dtype)
        streams = residual if residual.dim() == 3 else residual.unsqueeze(0)
        update = None
        if isinstance(delta, StreamUpdate):
            update = (delta.y, delta.mix, delta.out)
        elif isinstance(delta, AddedToResidual):
            delta = None
        elif delta is not None:
            if delta.dim() == 3 or streams.shape[0] != 1:
                raise ValueError("LayerNorm: a plain output can only be added to a single residual stream")
            if self._ones is None:
                self._ones = torch.ones(1, 1, dtype=torch.float32, device=residual.device)
            update = (delta, self._ones, self._ones.view(1))
        n = streams.shape[1] if rows is None else rows.shape[0]
        out = ctx.buffer(out_name, (n, self.size), out_dtype or ctx.act_dtype)
        if conv is not None:
            conv = (*conv, ctx.state_slots, ctx.attn_meta.context_lens)
        ops.hc_norm(streams, update=update, mix_in=mix_in, norm_weight=self.p(self.param), eps=self.eps, out=out, rows=rows,
                    conv=conv)
        return out


class GroupRMSNorm(Norm):
    """RMS norm in groups: a row is cut into ``groups`` equal consecutive parts, each part is divided by its own
    sqrt(mean(part^2) + eps), and the whole row is multiplied by a weight (``param`` names it on disk).  One group is the
    plain RMS norm.  Beside the usual ``forward`` (the model's last norm: nothing may be pending but a ``StreamCopy``) it has
    the two forms that a block with its norms BEHIND the sub-layers needs: ``add_normed`` (x <- x + norm(y)) and
    ``normalize_stream`` (x <- norm(x), the norm behind an embedding).  Both return the new stream in the working dtype as a
    ``StreamCopy``; in the float32 engine that is the stream itself."""
    capturable = True

    def __init__(self, size: int, eps: float, groups: int = 1, param: str = "weight"):
        super().__init__()
        if groups < 1 or size % groups:
            raise ValueError(f"GroupRMSNorm: {size} values do not split into {groups} equal groups")
        self.size, self.eps, self.groups, self.param = size, float(eps), int(groups), param

    def param_decls(self):
        return [ParamDecl(self.param, (self.size,), init="norm", role="vector")]

    @property
    def weight(self) -> torch.Tensor:
        return self.p(self.param)

    def _copy(self, residual, ctx):
        return None if ctx.act_dtype == torch.float32 else ctx.buffer("stream_copy", tuple(residual.shape), ctx.act_dtype)

    def add_normed(self, residual, y, ctx) -> StreamCopy:
        """``residual += norm(y)``; ``y`` [T, size] in any dtype the kernels know."""
        out = self._copy(residual, ctx)
        ops.group_norm(residual, y, self.weight, self.groups, self.eps, out)
        return StreamCopy(residual if out is None else out)

    def normalize_stream(self, residual, ctx) -> StreamCopy:
        out = self._copy(residual, ctx)
        ops.group_norm(residual, None, self.weight, self.groups, self.eps, out)
        return StreamCopy(residual if out is None else out)

    def forward(self, residual, delta, ctx, rows: Optional[torch.Tensor] = None, lazy: bool = False):
        if delta is not None and not isinstance(delta, (StreamCopy, AddedToResidual)):
            raise TypeError(f"GroupRMSNorm reads a stream that holds every sum; a pending {type(delta).__name__} cannot join it here")
        if rows is None:
            rows = ctx.buffer("all_rows", (residual.shape[0],), torch.int32)
            torch.arange(residual.shape[0], dtype=torch.int32, device=residual.device, out=rows)
        out = ctx.buffer("norm_out", (rows.shape[0], self.size), ctx.act_dtype)
        ops.group_norm(residual, None, self.weight, self.groups, self.eps, out, rows=rows)
        return out


register_norm("rmsnorm", RMSNorm)
register_norm("group_rmsnorm", GroupRMSNorm)
register_norm("layernorm", LayerNorm)
