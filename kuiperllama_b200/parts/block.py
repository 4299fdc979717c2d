"""How a layer's parts are arranged in a block."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..cache import CacheView
from .base import FeedForward, Mixer, Norm, NormedLazy, StepContext, StreamSink, register_arrangement


@register_arrangement("pre_norm")
class PreNormBlock:
    """x += mixer(norm1(x)); x += feed_forward(norm2(x))
    (ExiledOfCode/KuiperLLama kuiper/source/model/llama3.cpp:155-164, tools/model.py:200-203).

    The residual stream is float32.  A block receives the stream and a *pending* delta that
    the block before it has not added yet; every norm adds the pending delta while it reads
    the row, so no add runs as a kernel of its own.  The block returns the stream and its
    own feed-forward output as the next pending delta."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, feed_forward_norm: Norm, feed_forward: FeedForward):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    def forward(self, residual: torch.Tensor, pending, step: StepContext, cache: CacheView):
        # Where the step allows it (decode), a part that can add into the stream itself is given
        # the stream, and a part that can normalise the stream's rows itself is given them lazily.
        fuse = step.allow_stream_fusion
        after = step.next_norm                       # the norm that receives this block's pending result

        def sink_for(part, norm):
            ok = fuse and part.may_accumulate and norm is not None and getattr(norm, "accepts_accumulated", False)
            return StreamSink(residual, norm) if ok else None

        n = self.mixer_norm.forward(residual, pending, step.n_tokens)
        if isinstance(n, NormedLazy) and not self.mixer.accepts_lazy_norm:
            n = n.dense()
        step.residual_sink = sink_for(self.mixer, self.feed_forward_norm)
        mixed = self.mixer.forward(n, step, cache)
        n = self.feed_forward_norm.forward(residual, mixed, step.n_tokens)
        if isinstance(n, NormedLazy) and not self.feed_forward.accepts_lazy_norm:
            n = n.dense()
        step.residual_sink = sink_for(self.feed_forward, after)
        out = self.feed_forward.forward(n, step)
        step.residual_sink = None
        return residual, out
