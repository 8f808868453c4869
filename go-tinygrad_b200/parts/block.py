"""Arrangements of a layer's parts.

``pre_norm``: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(model/llama.go:1087-1097, 1311-1314, 1425).  Its parameters are the four
nested specs ``mixer_norm``, ``mixer``, ``feed_forward_norm`` and
``feed_forward``; the last two may be None for a layer that has a mixer only.
The additions are not done here: each update is left
pending on the residual stream and the next norm (of this layer, of the next
one, or the final one) adds it in float32 while it normalises -- unless the
part, offered the stream (`emit_update`), has added its update in its last
product's epilogue already and returns None.

``concat_projection``: x <- W [x | kept], a projection of the hidden state side
by side with a tensor an earlier part has kept for the step under the name
``source`` in the step's shared values (the token embedding keeps its output
as "embedding_output" when asked to).  It replaces the hidden state instead
of adding to it, holds no cache, and can stand anywhere in the schedule, as
often as wanted.  Parameters: ``hidden_size``, ``weight`` (tensor name,
[hidden, 2 hidden], the hidden state's columns first), ``source``.  The
reference has no such part.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..cache import CacheHandle
from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import Block, ResidualStream, Runtime, StepContext, register_part


def _hidden(stream: ResidualStream):
    """The hidden state as a value: the residual with its pending update added."""
    if stream.pending is None:
        return stream.residual.clone()
    return stream.residual + stream.pending.float()


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    sub_parts = (("mixer_norm", "norm"), ("mixer", "mixer"),
                 ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))
    optional_parts = ("feed_forward_norm", "feed_forward")

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheHandle) -> None:
        ctx.trace("hidden_in", lambda: _hidden(stream))
        x = self.mixer_norm.forward(stream, ctx)
        ctx.trace("normed", x)
        ctx.update_into = stream
        try:
            stream.pending = self.mixer.forward(x, ctx, cache)
            if stream.pending is not None:
                ctx.trace("o", stream.pending)
            if self.feed_forward is not None:
                x = self.feed_forward_norm.forward(stream, ctx)
                ctx.trace("mlp_input", x)
                stream.pending = self.feed_forward.forward(x, ctx)
                if stream.pending is not None:
                    ctx.trace("down", stream.pending)
        finally:
            ctx.update_into = None
        ctx.trace("hidden_post_ffn", lambda: _hidden(stream))


@register_part("block", "concat_projection")
class ConcatProjection(Block):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.weight_name = str(self.param("weight"))
        self.source = str(self.p.get("source") or "embedding_output")
        self.w: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.hidden, 2 * self.hidden))]

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.w = rt.matrix(tensors[self.weight_name])

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheHandle) -> None:
        kept = ctx.shared.get(self.source)
        if kept is None:
            raise ValueError(f"nothing was kept under {self.source!r} in this step for the projection to read")
        both = ctx.rt.empty(stream.residual.shape[0], 2 * self.hidden)
        ops.hidden_concat(stream.residual, stream.pending, kept, both)
        stream.pending = None
        ops.linear(both, self.w, stream.residual)
        ctx.trace("hidden_in", lambda: stream.residual.clone())
