"""The generation loop above the step function.

Requests are taken in order, as many at a time as the cache can hold; a batch's prompts run
in one step, then one token per live sequence per step.  A sequence ends at a stop token, at
its token limit or at the cache's length limit; it leaves the batch at once and its slot is
handed back, and when a batch is done the next one starts and reuses the slots.

ExiledOfCode/KuiperLLama's loop (demo/main.cpp:5-47) runs one sequence, feeds the prompt
token by token and counts positions; its stop rule is kept: the end-of-sentence test comes
before the token is appended (main.cpp:30-32), so the stop token is not part of the output,
and Llama 3 has two stop tokens (kuiper/source/op/encode.cpp:99-102,135-141), so stop ids are
a set.

The loop's decisions are separated from the device: ``run_requests`` talks to a *backend*
with four methods (alloc_slot, free_slot, prefill, decode), so they can be tested with a
fake backend on the CPU.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Iterable, List, Optional, Protocol, Sequence, Tuple

import torch

from ..cache import PAGE, pages_for
from ..sampling import Sampler, SamplingParams
from .step import Engine, SequenceInput


class Backend(Protocol):
    def alloc_slot(self) -> int: ...
    def free_slot(self, slot: int) -> None: ...
    def prefill(self, slots: List[int], prompts: List[Sequence[int]], request_ids: List[int]) -> List[int]: ...
    def decode(self, slots: List[int], last_tokens: List[int], request_ids: List[int], steps: List[int]) -> List[int]: ...


@dataclass
class RequestResult:
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""          # "stop", "length" (token limit) or "context" (cache length limit)


@dataclass
class GenerationStats:
    batches: int = 0
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_tokens: int = 0
    decode_steps: int = 0
    decode_seconds: float = 0.0


def tokens_held(prompt_len: int, max_new_tokens: int, max_seq_len: int) -> int:
    """Cache tokens a request may come to hold, rounded up to whole pages."""
    return pages_for(min(prompt_len + max_new_tokens, max_seq_len), PAGE) * PAGE


def next_batch(pending: Sequence[int], prompt_lens: Sequence[int], max_new_tokens: int, max_batch: int,
               token_budget: int, max_seq_len: int) -> List[int]:
    """The longest prefix of ``pending`` (request indices, in order) that fits: at most
    ``max_batch`` sequences whose page-rounded final lengths sum to at most ``token_budget``."""
    batch: List[int] = []
    used = 0
    for r in pending:
        need = tokens_held(prompt_lens[r], max_new_tokens, max_seq_len)
        if len(batch) >= max_batch or used + need > token_budget:
            break
        batch.append(r)
        used += need
    if not batch:
        r = pending[0]
        raise ValueError(f"request {r} ({prompt_lens[r]} prompt tokens) does not fit the cache "
                         f"({token_budget} tokens) even alone")
    return batch


def run_requests(backend: Backend, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                 stop_ids: Iterable[int] = (), include_stop: bool = False, max_batch: int = 64,
                 token_budget: int = 1 << 30, max_seq_len: int = 1 << 30,
                 stats: Optional[GenerationStats] = None) -> List[RequestResult]:
    stop = set(int(s) for s in stop_ids)
    stats = stats if stats is not None else GenerationStats()
    for i, p in enumerate(prompts):
        if len(p) < 1:
            raise ValueError(f"request {i} has an empty prompt")
        if len(p) >= max_seq_len and max_new_tokens > 0:
            raise ValueError(f"request {i}: a prompt of {len(p)} tokens leaves no room in a cache of {max_seq_len} per sequence")
    results = [RequestResult() for _ in prompts]
    if max_new_tokens <= 0:
        for r in results:
            r.finish_reason = "length"
        return results
    pending = list(range(len(prompts)))
    lens = [len(p) for p in prompts]
    while pending:
        batch = next_batch(pending, lens, max_new_tokens, max_batch, token_budget, max_seq_len)
        pending = pending[len(batch):]
        stats.batches += 1
        slots = [backend.alloc_slot() for _ in batch]
        t0 = time.perf_counter()
        new = backend.prefill(slots, [prompts[r] for r in batch], list(batch))
        stats.prefill_seconds += time.perf_counter() - t0
        stats.prefill_tokens += sum(lens[r] for r in batch)
        live: List[Tuple[int, int]] = list(zip(batch, slots))      # (request, slot)
        step = 0
        while True:
            still: List[Tuple[int, int]] = []
            last: List[int] = []
            for (r, slot), tok in zip(live, new):
                res = results[r]
                tok = int(tok)
                if tok in stop:
                    if include_stop:
                        res.tokens.append(tok)
                    res.finish_reason = "stop"
                else:
                    res.tokens.append(tok)
                    if len(res.tokens) >= max_new_tokens:
                        res.finish_reason = "length"
                    elif lens[r] + len(res.tokens) >= max_seq_len:
                        res.finish_reason = "context"    # the next token would not fit the cache
                if res.finish_reason:
                    backend.free_slot(slot)              # handed back at once; later batches reuse it
                else:
                    still.append((r, slot))
                    last.append(tok)
            live = still
            if not live:
                break
            step += 1
            t0 = time.perf_counter()
            new = backend.decode([s for _, s in live], last, [r for r, _ in live], [step] * len(live))
            stats.decode_seconds += time.perf_counter() - t0
            stats.decode_steps += 1
            stats.decode_tokens += len(live)
    return results


class EngineBackend:
    """The real backend: the step function plus a sampler.  Prefill wants the logits at
    each prompt's last token; decode brings one token per sequence."""

    def __init__(self, engine: Engine, sampler: Sampler):
        self.engine, self.sampler = engine, sampler
        self.device = engine.device

    def alloc_slot(self) -> int:
        return self.engine.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.engine.free_slot(slot)

    def _sample(self, logits: torch.Tensor, request_ids: List[int], steps: List[int]) -> List[int]:
        if self.sampler.greedy:
            ids = st = torch.empty(0, dtype=torch.int32, device=self.device)
        else:
            both = torch.tensor(request_ids + steps, dtype=torch.int32).to(self.device, non_blocking=True)
            ids, st = both[:len(request_ids)], both[len(request_ids):]
        return self.sampler.sample(logits, ids, st).tolist()          # device -> host: the step's result

    def prefill(self, slots, prompts, request_ids):
        logits = self.engine.step([SequenceInput(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        return self._sample(logits, list(request_ids), [0] * len(slots))

    def decode(self, slots, last_tokens, request_ids, steps):
        logits = self.engine.decode_step(slots, last_tokens)
        return self._sample(logits, list(request_ids), list(steps))
