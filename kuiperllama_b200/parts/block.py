"""How a layer's parts are arranged in a block."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..cache import CacheView
from .base import FeedForward, Mixer, Norm, StepContext, register_arrangement


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

    def forward(self, residual: torch.Tensor, pending: Optional[torch.Tensor], step: StepContext,
                cache: CacheView) -> Tuple[torch.Tensor, torch.Tensor]:
        n = self.mixer_norm.forward(residual, pending, step.n_tokens)
        mixed = self.mixer.forward(n, step, cache)
        n = self.feed_forward_norm.forward(residual, mixed, step.n_tokens)
        return residual, self.feed_forward.forward(n, step)
