"""The step function: one batch of sequences through the model, from the cache.

A step brings, for each sequence of the batch, its next tokens: a whole prompt of any
length at the batch's first step, then one token each.  It runs exactly those tokens as one
packed batch, appends their keys and values to each sequence's slot, and returns float32
logits at the wanted places.  (ExiledOfCode/KuiperLLama's counterpart is ``predict`` /
``forward`` for one token of one sequence, kuiper/source/model/llama3.cpp:641-649,146-166;
its prompt goes through token by token, demo/main.cpp:18-41.)

``Engine`` owns nothing numeric: it packs the batch, keeps the cache's lengths, and calls the
model.  Decode steps can be replayed from a CUDA graph (``use_graphs``): same kernels, same
buffers, launched as one graph per batch size.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import PAGE, CacheError, SequenceCache
from ..parts.base import StepContext
from .model import DecoderModel


class StepError(ValueError):
    """A batch the step function refuses (the message says why)."""


@dataclass
class SequenceInput:
    """One sequence's share of a step: the slot it lives in, its next tokens, and the
    places among these tokens whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


class _Staging:
    """Pinned host buffers and one device buffer that hold all of a step's integer inputs,
    so that a step costs one host-to-device copy.  The host side is a small ring: a buffer
    is written again only after the copy that read it has finished (its event), because the
    host runs ahead of the device."""

    RING = 4

    def __init__(self, capacity: int, device: torch.device):
        self.capacity = capacity
        cuda = device.type == "cuda"
        self.hosts = [torch.zeros(capacity, dtype=torch.int32, pin_memory=cuda) for _ in range(self.RING)]
        self.events = [torch.cuda.Event() if cuda else None for _ in range(self.RING)]
        self.used = [False] * self.RING
        self.turn = 0
        self.dev = torch.zeros(capacity, dtype=torch.int32, device=device)

    def upload(self, flat) -> torch.Tensor:
        """``flat``: a list of ints, or a list of int32 numpy arrays that are laid end to end."""
        i = self.turn
        self.turn = (i + 1) % self.RING
        if self.used[i] and self.events[i] is not None:
            self.events[i].synchronize()
        if flat and isinstance(flat[0], np.ndarray):
            view = self.hosts[i].numpy()
            n = 0
            for a in flat:
                view[n:n + a.size] = a
                n += a.size
        else:
            n = len(flat)
            self.hosts[i][:n] = torch.tensor(flat, dtype=torch.int32)
        self.dev[:n].copy_(self.hosts[i][:n], non_blocking=True)
        if self.events[i] is not None:
            self.events[i].record()
            self.used[i] = True
        return self.dev


def context_class(max_context: int) -> int:
    """The class of a step by its longest sequence: 0 up to 16 cache pages, then one class per
    doubling.  A captured decode step is replayed only for steps of its own class, so a part may
    plan a decode launch by ``step.context_class`` (into how many pieces it cuts a sequence's keys,
    say); what it plans by ``max_context`` itself would go stale inside a graph."""
    pages = -(-max(int(max_context), 1) // PAGE)
    return max(0, (pages - 1).bit_length() - 4)


class _DecodeGraph:
    """One captured decode step for a fixed number of sequences and a context class.  The kernels read their
    integer inputs from the engine's staging buffer and the cache's block tables, which keep
    their addresses; a replay runs the step on whatever those hold."""

    def __init__(self, graph: "torch.cuda.CUDAGraph", logits: torch.Tensor, staging_ptr: int, launches: int):
        self.graph, self.logits, self.staging_ptr, self.launches = graph, logits, staging_ptr, launches


class Engine:
    # A captured step keeps its own activations and logits (64 sequences of a 128k vocabulary: 33 MB);
    # beyond this many the one replayed longest ago is dropped and captured again if it comes back.
    MAX_GRAPHS = 48
    # Small steps that are not decode steps (a short prompt, a chunk of one) are captured too, since the
    # host needs longer to launch their kernels one by one than the device to run them (8B shape, 128
    # tokens: 161 us of host time per layer, about 110 us of kernels).  Their rows are padded to a
    # multiple of 64, and a captured step serves every step of as many sequences, padded rows and
    # wanted places.
    SMALL_STEP_TOKENS = 512
    SMALL_STEP_SEQS = 8
    MAX_STEP_GRAPHS = 16

    def __init__(self, model: DecoderModel, cache: SequenceCache, use_graphs: bool = False):
        self.model = model
        self.cache = cache
        self.device = model.runtime.device
        self.use_graphs = use_graphs
        self._staging: Optional[_Staging] = None
        self._graphs: Dict[Tuple[int, int], _DecodeGraph] = {}        # (sequences, context class) -> captured step
        self._step_graphs: Dict[Tuple[int, int, int], _DecodeGraph] = {}   # (sequences, padded rows, wanted places) -> captured small step

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    # ------------------------------------------------------------------ packing
    def _pack(self, inputs: Sequence[SequenceInput], pad_rows: int) -> Tuple[StepContext, torch.Tensor, int]:
        if not inputs:
            raise StepError("an empty batch")
        vocab = self.model.spec.vocab_size
        slots, starts, news, token_arrays = [], [], [], []
        seen = set()
        for s in inputs:
            if not self.cache.slots.is_held(s.slot):
                raise StepError(f"slot {s.slot} is not held by a sequence")
            if s.slot in seen:
                raise StepError(f"slot {s.slot} appears twice in one step")
            seen.add(s.slot)
            n = len(s.tokens)
            if n < 1:
                raise StepError(f"the sequence in slot {s.slot} brings no token")
            for w in s.want:
                if not 0 <= w < n:
                    raise StepError(f"slot {s.slot}: wanted place {w} is outside its {n} tokens")
            toks = np.asarray(s.tokens, dtype=np.int64)
            lo, hi = int(toks.min()), int(toks.max())
            if lo < 0 or hi >= vocab:
                raise StepError(f"slot {s.slot}: token id {lo if lo < 0 else hi} is outside the vocabulary of {vocab}")
            token_arrays.append(toks.astype(np.int32))
            slots.append(s.slot)
            starts.append(self.cache.lengths[s.slot])
            news.append(n)
        n_real = sum(news)
        n_rows = n_real + pad_rows
        n_seqs = len(inputs)
        n_want = sum(len(s.want) for s in inputs)
        for s, st, n in zip(inputs, starts, news):
            try:
                self.cache.reserve(s.slot, st + n)
            except CacheError as e:
                raise StepError(str(e)) from None
        self.cache.flush_tables()

        # layout of the staging buffer: ids | positions | token_slot | slots | starts | news | cu | want
        total = 3 * n_rows + 3 * n_seqs + (n_seqs + 1) + n_want
        if self._staging is None or self._staging.capacity < total:
            self._staging = _Staging(max(total * 2, 1 << 16), self.device)
        i32 = np.int32
        pad = np.zeros(pad_rows, dtype=i32)
        cu = np.zeros(n_seqs + 1, dtype=i32)
        np.cumsum(news, out=cu[1:])
        want = [cu[j] + np.asarray(s.want, dtype=i32) for j, s in enumerate(inputs) if len(s.want)]
        flat = (token_arrays + [pad]
                + [np.arange(st, st + n, dtype=i32) for st, n in zip(starts, news)] + [pad]
                + [np.full(n, sl, dtype=i32) for sl, n in zip(slots, news)] + [np.full(pad_rows, -1, dtype=i32)]
                + [np.asarray(slots, dtype=i32), np.asarray(starts, dtype=i32), np.asarray(news, dtype=i32), cu] + want)
        d = self._staging.upload(flat)
        o = 0

        def take(k: int) -> torch.Tensor:
            nonlocal o
            v = d[o:o + k]
            o += k
            return v

        ctx = StepContext(
            n_tokens=n_rows, n_seqs=n_seqs, token_ids=take(n_rows), positions=take(n_rows), token_slot=take(n_rows),
            seq_slots=take(n_seqs), seq_starts=take(n_seqs), seq_new=take(n_seqs), cu_tokens=take(n_seqs + 1),
            is_decode=all(n == 1 for n in news), max_new=max(news),
            max_context=max(st + n for st, n in zip(starts, news)),
            context_class=context_class(max(st + n for st, n in zip(starts, news))),
            host_slots=slots, host_starts=starts, host_new=news)
        want_rows = take(n_want)
        return ctx, want_rows, n_want

    # ------------------------------------------------------------------ the step
    def step(self, inputs: Sequence[SequenceInput], pad_rows: int = 0) -> Optional[torch.Tensor]:
        """Run one step.  Returns float32 logits [wanted, vocab] in the order of ``inputs``
        and of each ``want`` (None when nothing is wanted).  ``pad_rows`` appends rows that
        belong to no sequence; they change no result."""
        if self.use_graphs and pad_rows == 0 and self._is_small_step(inputs):
            return self._small_step(inputs)
        ctx, want_rows, n_want = self._pack(inputs, pad_rows)
        residual, pending = self.model.hidden_states(ctx, self.cache)
        for s, st, n in zip(inputs, ctx.host_starts, ctx.host_new):
            self.cache.lengths[s.slot] = st + n
        if n_want == 0:
            return None
        return self.model.logits(residual, pending, want_rows)

    def _is_small_step(self, inputs: Sequence[SequenceInput]) -> bool:
        if not 1 <= len(inputs) <= self.SMALL_STEP_SEQS:
            return False
        n = sum(len(s.tokens) for s in inputs)
        return n <= self.SMALL_STEP_TOKENS and any(len(s.tokens) > 1 for s in inputs)

    def _small_step(self, inputs: Sequence[SequenceInput]) -> Optional[torch.Tensor]:
        """A small step through a CUDA graph: the rows padded to a multiple of 64, the attention's
        grid sized for sequences of up to that many new tokens, everything else read from the staging
        buffer and the block tables as in any step.  The first step of a key runs kernel by kernel
        and is then captured.  The logits are a copy (the graph's own buffer is written by the next
        replay)."""
        from ..csrc import ops
        n_real = sum(len(s.tokens) for s in inputs)
        rows = -(-n_real // PAGE) * PAGE
        ctx, want_rows, n_want = self._pack(inputs, rows - n_real)
        ctx.max_new = rows                                # every length a replay may bring
        key = (ctx.n_seqs, rows, n_want)
        g = self._step_graphs.get(key)
        if g is not None and g.staging_ptr != self._staging.dev.data_ptr():
            self._step_graphs.clear()                     # the staging buffer moved: captured addresses are stale
            self._graphs.clear()
            g = None
        if g is None:
            residual, pending = self.model.hidden_states(ctx, self.cache)
            logits = self.model.logits(residual, pending, want_rows) if n_want else None
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            with torch.cuda.graph(graph):
                r2, p2 = self.model.hidden_states(ctx, self.cache)
                static_logits = self.model.logits(r2, p2, want_rows) if n_want else None
            captured = ops.launch_count - before
            ops.launch_count = before
            self._step_graphs[key] = _DecodeGraph(graph, static_logits, self._staging.dev.data_ptr(), captured)
            while len(self._step_graphs) > self.MAX_STEP_GRAPHS:
                self._step_graphs.pop(next(iter(self._step_graphs)))
        else:
            self._step_graphs[key] = self._step_graphs.pop(key)      # most recently used last
            g.graph.replay()
            ops.launch_count += g.launches
            logits = g.logits.clone() if n_want else None
        for s, st, n in zip(inputs, ctx.host_starts, ctx.host_new):
            self.cache.lengths[s.slot] = st + n
        return logits

    def decode_step(self, slots: Sequence[int], tokens) -> torch.Tensor:
        """One token for each of the given sequences; logits [len(slots), vocab].  ``tokens`` are
        token ids on the host, or an int32 tensor on the device (the sampler's output of the step
        before, which the host need not have seen yet).

        With ``use_graphs`` the step of a batch size (and of a class of context lengths, see
        ``context_class``) is captured in a CUDA graph the first time it runs and replayed
        afterwards: the same kernels on the same buffers with one launch.  The logits tensor of a
        replayed step is the graph's own output buffer; it is overwritten by the next decode step
        of the same batch size and class."""
        on_device = isinstance(tokens, torch.Tensor)
        n = len(slots)
        key, g = None, None
        if self.use_graphs:
            try:
                key = (n, context_class(max(self.cache.lengths[s] for s in slots) + 1))
            except (IndexError, KeyError, TypeError, ValueError):
                key = (n, 0)                                  # a bad slot: the ordinary path below says so
            g = self._graphs.get(key)
            if g is not None:
                self._graphs[key] = self._graphs.pop(key)     # most recently used last
        if g is not None and self._staging is not None and g.staging_ptr == self._staging.dev.data_ptr():
            return self._replay(g, list(slots), tokens if on_device else [int(t) for t in tokens])
        if on_device:
            tokens = tokens.tolist()                      # no graph for this size yet: the ordinary way, through the host
        if not self.use_graphs:
            return self.step([SequenceInput(s, [int(t)], [0]) for s, t in zip(slots, tokens)])
        from ..csrc import ops
        inputs = [SequenceInput(s, [int(t)], [0]) for s, t in zip(slots, tokens)]
        ctx, want_rows, _ = self._pack(inputs, 0)
        if g is not None:                                 # the staging buffer moved: captured addresses are stale
            self._graphs.clear()
            self._step_graphs.clear()
            g = None
        if g is None:
            # The first step of this size runs eagerly (it also warms every kernel up); then the
            # same calls are captured for the steps that follow.  Capturing launches nothing.
            residual, pending = self.model.hidden_states(ctx, self.cache)
            logits = self.model.logits(residual, pending, want_rows)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            with torch.cuda.graph(graph):
                r2, p2 = self.model.hidden_states(ctx, self.cache)
                static_logits = self.model.logits(r2, p2, want_rows)
            captured = ops.launch_count - before
            ops.launch_count = before                     # captured calls are not launches; replays are counted below
            self._graphs[(n, ctx.context_class)] = _DecodeGraph(graph, static_logits, self._staging.dev.data_ptr(), captured)
            while len(self._graphs) > self.MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
        else:
            g.graph.replay()
            ops.launch_count += g.launches
            logits = g.logits
        for s, st in zip(inputs, ctx.host_starts):
            self.cache.lengths[s.slot] = st + 1
        return logits

    def graph_sizes(self) -> List[int]:
        """The batch sizes whose decode step has been captured (in any context class)."""
        return sorted({n for n, _ in self._graphs})

    def _replay(self, g: _DecodeGraph, slots: List[int], tokens) -> torch.Tensor:
        """The short way through a decode step whose graph exists: the same checks and the same
        staging layout as ``_pack`` for one token per sequence, then one graph launch.  Token
        ids that are already on the device are copied into place there (the embedding kernel
        flags an id outside the vocabulary)."""
        from ..csrc import ops
        n = len(slots)
        cache, lengths = self.cache, self.cache.lengths
        on_device = isinstance(tokens, torch.Tensor)
        if len(set(slots)) != n:
            raise StepError("a slot appears twice in one step")
        if on_device:
            if tokens.numel() != n or tokens.dtype != torch.int32 or not tokens.is_cuda:
                raise StepError("device token ids must be an int32 CUDA tensor with one id per sequence")
        elif min(tokens) < 0 or max(tokens) >= self.model.spec.vocab_size:
            raise StepError(f"a token id is outside the vocabulary of {self.model.spec.vocab_size}")
        starts = []
        for s in slots:
            if not cache.slots.is_held(s):
                raise StepError(f"slot {s} is not held by a sequence")
            st = lengths[s]
            if st % PAGE == 0 or st + 1 > cache.max_seq_len:      # a new page, or the limit: let the cache decide
                try:
                    cache.reserve(s, st + 1)
                except CacheError as e:
                    raise StepError(str(e)) from None
            starts.append(st)
        cache.flush_tables()
        # ids | positions | token_slot | slots | starts | news | cu | want
        ids = [0] * n if on_device else tokens
        dev = self._staging.upload(ids + starts + slots + slots + starts + [1] * n + list(range(n + 1)) + list(range(n)))
        if on_device:
            dev[:n].copy_(tokens)
        g.graph.replay()
        ops.launch_count += g.launches
        for s, st in zip(slots, starts):
            lengths[s] = st + 1
        return g.logits

    def check_device_errors(self) -> None:
        """Synchronises, reads the device's two report words in one copy and raises if a kernel
        gave up a bounded wait (``KernelError``: the step's results are not valid) or met a token
        id outside the vocabulary (``StepError``).  What was set is cleared."""
        from ..csrc import ops
        try:
            ops.check_device_words(self.device)
        except ops.TokenIdError as e:
            raise StepError(str(e)) from None
