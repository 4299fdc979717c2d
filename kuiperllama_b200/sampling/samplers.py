"""Choosing the next token from float32 logits, on the device.

ExiledOfCode/KuiperLLama's C++ engine samples with argmax only
(kuiper/source/sampler/argmax_sampler.cpp:5-13); its Python model also has temperature and
top-k (tools/model.py:327-339: temperature 0 means the most likely token; otherwise
logits / temperature, an optional cut to the k largest, softmax, one draw).  Both are here.
The draw uses a counter-based generator keyed by (seed, request id, step), so a request's
tokens do not depend on which other requests share its batch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..csrc import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0          # 0: greedy (argmax, the lowest index among equal logits)
    top_k: Optional[int] = None       # keep the logits not below the k-th largest
    seed: int = 0

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must not be negative, got {self.temperature}")
        if self.top_k is not None and self.top_k < 1:
            raise ValueError(f"top_k must be at least 1, got {self.top_k}")


def uniform_from_counter(seed: int, request: int, step: int) -> float:
    """The draw in [0, 1) the sampling kernel makes for (seed, request, step); kept here so
    that hosts can reproduce a run.  A 64-bit mix of the three, top 24 bits."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & mask
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & mask
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, params: SamplingParams):
        params.validate()
        self.params = params

    @property
    def greedy(self) -> bool:
        return self.params.temperature == 0.0

    def sample(self, logits: torch.Tensor, request_ids: torch.Tensor, steps: torch.Tensor,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits: float32 [rows, vocab] on the device; request_ids, steps: int32 [rows].
        Returns int32 [rows] on the device."""
        rows = logits.shape[0]
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        if self.greedy:
            ops.argmax_rows(logits, out)
        else:
            ops.sample_rows(logits, self.params.temperature, self.params.top_k or 0, self.params.seed,
                            request_ids, steps, out)
        return out
