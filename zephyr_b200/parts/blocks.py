"""Arrangements of a layer's parts around the residual stream.

``prenorm_residual``: r = x + mixer(norm1(x)); x' = r + ffn(norm2(r)), the sums in float32
(reference: src/model/causal_lm/qwen3.cpp:79-88).  Each sum is folded into the norm that follows
it, so the block hands its last summand on as ``pending``.
"""

from __future__ import annotations

from typing import Mapping

from ..config.spec import LayerCall
from .base import Block, FeedForward, Mixer, Norm, ResidualStream, StepContext, register_block
from .fused import BlockPlan


class PreNormResidual(Block):
    graph_safe = True

    norm_names = ("mixer", "feed_forward")

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Mapping[str, Norm]):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)
        self.mixer_norm = norms["mixer"]
        self.feed_forward_norm = norms["feed_forward"]

    def forward(self, stream: ResidualStream, ctx: StepContext, call: LayerCall) -> ResidualStream:
        if stream.pending is None:
            normed = self.mixer_norm.forward(stream.hidden)
        else:
            normed = self.mixer_norm.add_forward(stream.hidden, stream.pending)
        mixed = self.mixer.forward(normed, ctx, call)
        normed = self.feed_forward_norm.add_forward(stream.hidden, mixed)
        stream.pending = self.feed_forward.forward(normed)
        return stream


    def chain_plan(self) -> BlockPlan | None:
        mixer_norm, ffn_norm = self.mixer_norm.as_rms_scale(), self.feed_forward_norm.as_rms_scale()
        gated = self.feed_forward.as_gated_products()
        if mixer_norm is None or ffn_norm is None or gated is None:
            return None
        return BlockPlan(self.mixer, mixer_norm, ffn_norm, gated[0], gated[1])


register_block("prenorm_residual", PreNormResidual)
