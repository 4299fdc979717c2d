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
    """What the loop needs of an engine.  ``prefill`` and ``decode`` return a *handle* to the
    tokens they sampled (one per sequence, in the order given); ``read`` waits for a handle's
    tokens and returns them as a list.  ``decode`` takes the handle of the step before and,
    for each of its sequences, the place of that sequence's token in it, so a backend can run
    a step before the host has seen the tokens that feed it."""
    def alloc_slot(self) -> int: ...
    def free_slot(self, slot: int) -> None: ...
    def prefill(self, slots: List[int], prompts: List[Sequence[int]], request_ids: List[int]): ...
    def decode(self, slots: List[int], previous, take: List[int], request_ids: List[int], steps: List[int]): ...
    def read(self, handle) -> List[int]: ...
    def select(self, handle, keep: List[int]): ...      # the handle of a subset, in the order of `keep`
    # Only when the loop is asked for log-probabilities or logits: after ``read(handle)``, for every
    # sequence of the handle (logprob of its token or None, its logits row or None).
    def details(self, handle) -> List[tuple]: ...


@dataclass
class RequestResult:
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""          # "stop", "length" (token limit) or "context" (cache length limit)
    logprobs: Optional[List[float]] = None     # log softmax(logits)[token] of every token of ``tokens``, if asked for
    logits: Optional[list] = None              # the float32 logits row every token was chosen from, if asked for


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
                 stats: Optional[GenerationStats] = None, want_details: bool = False) -> List[RequestResult]:
    """Run every request to its end and return the results in request order.  Whatever happens
    (an exception of the backend included), the slots of the batch under way are handed back."""
    stop = set(int(s) for s in stop_ids)
    stats = stats if stats is not None else GenerationStats()
    for i, p in enumerate(prompts):
        if len(p) < 1:
            raise ValueError(f"request {i} has an empty prompt")
        if len(p) >= max_seq_len and max_new_tokens > 0:
            raise ValueError(f"request {i}: a prompt of {len(p)} tokens leaves no room in a cache of {max_seq_len} per sequence")
    results = [RequestResult() for _ in prompts]
    if want_details:
        for r in results:
            r.logprobs, r.logits = [], []
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
        held: List[int] = []
        try:
            for _ in batch:
                held.append(backend.alloc_slot())
            slots = list(held)
            t0 = time.perf_counter()
            new = backend.prefill(slots, [prompts[r] for r in batch], list(batch))
            stats.prefill_tokens += sum(lens[r] for r in batch)
            live: List[Tuple[int, int]] = list(zip(batch, slots))      # (request, slot), in the order of `new`
            step = 0
            t_decode = None
            while True:
                # The next step is started before this step's tokens are read: it only needs them on
                # the device.  A sequence that is certain to end with the token being read (its token
                # limit or the cache's length limit) is left out; one that ends with a stop token has
                # run one step for nothing, and that step's token for it is dropped.
                ahead, take = [], []
                for j, (r, slot) in enumerate(live):
                    made = len(results[r].tokens) + 1
                    if made < max_new_tokens and lens[r] + made < max_seq_len:
                        ahead.append((r, slot))
                        take.append(j)
                nxt = None
                if ahead:
                    step += 1
                    nxt = backend.decode([s for _, s in ahead], new, take, [r for r, _ in ahead], [step] * len(ahead))
                    stats.decode_steps += 1
                tokens = backend.read(new)
                details = backend.details(new) if want_details else None
                if t_decode is None:
                    stats.prefill_seconds += time.perf_counter() - t0
                    t_decode = time.perf_counter()
                else:
                    stats.decode_tokens += len(live)
                finished = set()
                for j, ((r, slot), tok) in enumerate(zip(live, tokens)):
                    res = results[r]
                    tok = int(tok)
                    if details is not None and (tok not in stop or include_stop):
                        res.logprobs.append(details[j][0])
                        res.logits.append(details[j][1])
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
                        finished.add(r)
                        backend.free_slot(slot)              # handed back at once; later batches reuse it
                        held.remove(slot)
                if nxt is None or all(r in finished for r, _ in ahead):
                    if nxt is not None:
                        backend.read(nxt)                    # let the step that ran for nothing finish
                    break
                if any(r in finished for r, _ in ahead):
                    # the step ahead ran for these too: go on with the others, from their places in it
                    keep = [j for j, (r, _) in enumerate(ahead) if r not in finished]
                    new = backend.select(nxt, keep)
                    live = [ahead[j] for j in keep]
                else:
                    new, live = nxt, ahead
        finally:
            for slot in held:                                # only after an exception: nothing may stay held
                try:
                    backend.free_slot(slot)
                except Exception:
                    pass
        if t_decode is not None:
            stats.decode_seconds += time.perf_counter() - t_decode
    return results


class EngineBackend:
    """The real backend: the step function plus a sampler.  Prefill wants the logits at
    each prompt's last token; decode brings one token per sequence.  With ``logprobs`` /
    ``logits`` every step also leaves log softmax(logits)[token] (a kernel of this package) /
    a host copy of the float32 logits rows for ``details``."""

    def __init__(self, engine: Engine, sampler: Sampler, logprobs: bool = False, logits: bool = False):
        self.engine, self.sampler = engine, sampler
        self.device = engine.device
        self.want_logprobs, self.want_logits = logprobs, logits

    def alloc_slot(self) -> int:
        return self.engine.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.engine.free_slot(slot)

    def _sample(self, logits: torch.Tensor, request_ids: List[int], steps: List[int]) -> "_Tokens":
        if self.sampler.greedy:
            ids = st = torch.empty(0, dtype=torch.int32, device=self.device)
        else:
            both = torch.tensor(request_ids + steps, dtype=torch.int32).to(self.device, non_blocking=True)
            ids, st = both[:len(request_ids)], both[len(request_ids):]
        tokens = self.sampler.sample(logits, ids, st)
        logprobs = None
        if self.want_logprobs:
            from ..csrc import ops
            logprobs = ops.token_logprob(logits, tokens)
        # the logits of a replayed graph are overwritten by the next step of that size: the copy to
        # the host is queued here, before that step can be
        return _Tokens(tokens, logprobs, logits if self.want_logits else None)

    def prefill(self, slots, prompts, request_ids):
        logits = self.engine.step([SequenceInput(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        return self._sample(logits, list(request_ids), [0] * len(slots))

    def decode(self, slots, previous, take, request_ids, steps):
        tokens = previous.device_tokens if take == list(range(previous.n)) else self.select(previous, take).device_tokens
        logits = self.engine.decode_step(slots, tokens)
        return self._sample(logits, list(request_ids), list(steps))

    def read(self, handle):
        return handle.read()

    def details(self, handle):
        return handle.details()

    def select(self, handle, keep):
        idx = torch.tensor(keep, dtype=torch.int64).to(self.device, non_blocking=True)
        return _Tokens(handle.device_tokens.index_select(0, idx), keep=keep, parent=handle)


class _Tokens:
    """Sampled tokens of one step: on the device for the step that follows, and on their way to
    pinned host memory (the device-to-host read of the step's result) for the loop; with them,
    if asked for, the tokens' log-probabilities and the logits rows."""

    def __init__(self, device_tokens: torch.Tensor, logprobs: Optional[torch.Tensor] = None,
                 logits: Optional[torch.Tensor] = None, keep: Optional[List[int]] = None, parent: Optional["_Tokens"] = None):
        self.device_tokens = device_tokens
        self.n = device_tokens.numel()
        self.host = torch.empty(self.n, dtype=torch.int32, pin_memory=True)
        self.host.copy_(device_tokens, non_blocking=True)
        self.keep, self.parent = keep, parent
        self.host_logprobs = self.host_logits = None
        if logprobs is not None:
            self.host_logprobs = torch.empty(self.n, dtype=torch.float32, pin_memory=True)
            self.host_logprobs.copy_(logprobs, non_blocking=True)
        if logits is not None:
            self.host_logits = torch.empty(tuple(logits.shape), dtype=torch.float32, pin_memory=True)
            self.host_logits.copy_(logits, non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record()

    def read(self) -> List[int]:
        self.event.synchronize()
        return self.host.tolist()

    def details(self) -> List[tuple]:
        """(log-probability or None, logits row or None) for every sequence, after ``read``."""
        if self.parent is not None:                       # a subset of a step that was read already
            rows = self.parent.details()
            return [rows[j] for j in self.keep]
        self.event.synchronize()
        lp = self.host_logprobs.tolist() if self.host_logprobs is not None else [None] * self.n
        lg = [self.host_logits[i].clone() for i in range(self.n)] if self.host_logits is not None else [None] * self.n
        return list(zip(lp, lg))
