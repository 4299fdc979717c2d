"""The cache of a model: a slot for each live sequence, paged keys and values for every
execution of a layer that asks for them, and fixed-size state per slot.

* A *slot* belongs to one sequence from its first token until the sequence ends; then it is
  handed back and the next sequence reuses it, with the old contents still in the pages.
* Keys and values live in pages of ``PAGE`` tokens.  Executions of layers whose requests
  are equal (kind, kv heads, head size, window) form a *group*; each group has storage, a
  page pool and a block table of its own, so layers with different needs do not share a
  layout.  The storage of one execution is ``[pages, kv_heads, PAGE, head_dim]``.
* A group whose mixers read only a *window* of the most recent keys holds only the pages that
  the window still touches: before a step, the pages of a sequence that lie wholly below
  ``length - window + 1`` go back to the group's pool (no query of this or a later step reads
  them), so such a group can be given a smaller pool (``window_step_tokens``).
* Beside the pages every execution may ask for per-slot state of a fixed shape (a
  recurrent mixer's state, for instance).  It is zeroed when a slot is handed out.  The
  dense Llama decoder asks for none.

ExiledOfCode/KuiperLLama keeps two float32 tensors [layers, seq_len, kv_dim] for its single
sequence (kuiper/source/model/llama3.cpp:468-474, model.cpp:221-238).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .allocators import CacheError, FreeList, pages_for

PAGE = 64      # tokens per page; the kernels are compiled for the same number


@dataclass(frozen=True)
class KVRequest:
    """Token-indexed storage a mixer asks for.  ``kind`` names a registered storage class
    (``register_cache_kind``); "full": keys are stored by position in pages.
    ``window`` is the number of most recent keys the mixer reads (None: all); with a window
    the pages that no query can reach any more are given back while the sequence grows."""
    kv_heads: int
    head_dim: int
    kind: str = "full"
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """Per-slot state of a fixed shape that a mixer asks for."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheView:
    """What one execution of a layer sees of the cache."""
    k: Optional[torch.Tensor]             # [pages, kv_heads, PAGE, head_dim] or None
    v: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]   # int32 [slots, blocks_per_seq] of the group
    state: Optional[torch.Tensor]         # [slots, *shape] or None
    writable: bool                        # False: the execution reads another one's cache


_KINDS: Dict[str, type] = {}


def register_cache_kind(name: str):
    """Class decorator: token-indexed storage of the kind ``KVRequest.kind`` names.  The class is
    built as ``cls(request, entries, max_tokens_pages, n_slots, blocks_per_seq, dtype, device,
    window_step_tokens)`` for the schedule entries whose requests are equal, and offers

    * ``reserve(slot, old_length, new_length)``: room for the sequence to grow (raises CacheError),
    * ``release(slot)``: everything the sequence holds goes back,
    * ``flush()``: bring device-side tables up to date on the current stream,
    * ``view(j) -> (k, v, block_table)``: what execution ``entries[j]`` sees,
    * ``held() -> int`` and ``pool_size() -> int`` for the accounting, ``bytes() -> int``.
    """
    def deco(cls: type) -> type:
        _KINDS[name] = cls
        return cls
    return deco


def cache_kind(name: str) -> type:
    try:
        return _KINDS[name]
    except KeyError:
        raise CacheError(f"cache kind {name!r} is not known (known: {', '.join(sorted(_KINDS))})") from None


@register_cache_kind("full")
class PagedGroup:
    """Keys and values stored by position in pages of ``PAGE`` tokens,
    ``[executions, pages, kv_heads, PAGE, head_dim]``, with a block table per slot.  With a
    ``window`` in the request, pages that no query can reach any more go back to the pool while
    the sequence grows."""

    def __init__(self, request: KVRequest, entries: List[int], n_pages: int, n_slots: int, blocks_per_seq: int,
                 dtype: torch.dtype, device: torch.device, window_step_tokens: Optional[int] = None):
        self.request = request
        self.entries = entries
        if request.window is not None and window_step_tokens is not None:
            # the window's keys and the step's new tokens, both possibly straddling page borders
            per_slot = pages_for(request.window + window_step_tokens, PAGE) + 1
            n_pages = max(1, min(n_pages, n_slots * per_slot))
        self.pages = FreeList(n_pages, "page")
        self.blocks_per_seq = blocks_per_seq
        shape = (len(entries), n_pages, request.kv_heads, PAGE, request.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        # Pageable on purpose: a copy from pageable memory is staged before the call returns,
        # so the host may rewrite a row (a slot that is reused) while an earlier step's copy
        # is still queued on the device.
        self.table_host = torch.zeros((n_slots, blocks_per_seq), dtype=torch.int32)
        self.table = torch.zeros((n_slots, blocks_per_seq), dtype=torch.int32, device=device)
        # a sequence's pages by block index; a block below the window that was given back is -1
        self.slot_pages: List[List[int]] = [[] for _ in range(n_slots)]
        self.first_block: List[int] = [0] * n_slots            # blocks below this one were given back
        self.dirty: set = set()

    def pages_of(self, slot: int) -> List[int]:
        """The pages the sequence in ``slot`` holds now."""
        return [p for p in self.slot_pages[slot] if p >= 0]

    def reserve(self, slot: int, old_length: int, new_length: int) -> None:
        have = self.slot_pages[slot]
        if self.request.window is not None:
            # the first key any query of this step (positions old_length and up) or of a later
            # one reads is old_length - window + 1: whole blocks below it go back to the pool
            keep_from = min(max(0, old_length - self.request.window + 1) // PAGE, len(have))
            for b in range(self.first_block[slot], keep_from):
                self.pages.give_back(have[b])
                have[b] = -1
            self.first_block[slot] = max(self.first_block[slot], keep_from)
        need = pages_for(new_length, PAGE)
        if need > len(have):
            fresh = self.pages.take_many(need - len(have))
            for p in fresh:
                self.table_host[slot, len(have)] = p
                have.append(p)
            self.dirty.add(slot)

    def release(self, slot: int) -> None:
        for p in reversed(self.pages_of(slot)):
            self.pages.give_back(p)
        self.slot_pages[slot] = []
        self.first_block[slot] = 0

    def flush(self) -> None:
        if not self.dirty:
            return
        lo, hi = min(self.dirty), max(self.dirty) + 1
        self.table[lo:hi].copy_(self.table_host[lo:hi], non_blocking=True)
        self.dirty.clear()

    def view(self, j: int):
        return self.k[j], self.v[j], self.table

    def held(self) -> int:
        return self.pages.held()

    def pool_size(self) -> int:
        return self.pages.n

    def bytes(self) -> int:
        return self.k.numel() * self.k.element_size() * 2


class SequenceCache:
    """``max_tokens`` is the most tokens that live sequences hold at any time, each
    sequence's count rounded up to a multiple of ``PAGE``; it sizes every group's pool.
    ``max_seq_len`` bounds one sequence.  ``kv_requests[i]`` / ``state_requests[i]`` are the
    requests of schedule entry i (None: nothing); ``cache_from[i]`` names an earlier entry
    whose storage entry i reads instead of owning some.  ``window_step_tokens``: the most tokens
    a sequence brings in one step, if the caller can promise one; the pool of a group with a
    window is then sized for ``window + window_step_tokens`` tokens per slot instead of for
    ``max_tokens``."""

    def __init__(self, kv_requests: Sequence[Optional[KVRequest]],
                 state_requests: Sequence[Optional[StateRequest]], cache_from: Sequence[Optional[int]],
                 max_tokens: int, max_seq_len: int, dtype: torch.dtype, device, max_slots: Optional[int] = None,
                 window_step_tokens: Optional[int] = None):
        if max_tokens < PAGE:
            raise CacheError(f"max_tokens {max_tokens} is less than one page of {PAGE} tokens")
        self.device = torch.device(device)
        self.dtype = dtype
        self.n_pages = max_tokens // PAGE
        self.max_seq_len = min(max_seq_len, self.n_pages * PAGE)
        self.n_slots = self.n_pages if max_slots is None else max(1, min(max_slots, self.n_pages))
        self.blocks_per_seq = pages_for(self.max_seq_len, PAGE)
        self.slots = FreeList(self.n_slots, "slot")
        self.lengths: List[int] = [0] * self.n_slots
        self.cache_from = list(cache_from)

        # group the executions that own storage by their request
        by_request: Dict[KVRequest, List[int]] = {}
        for i, (req, src) in enumerate(zip(kv_requests, cache_from)):
            if req is not None and src is None:
                by_request.setdefault(req, []).append(i)
        self.window_step_tokens = window_step_tokens
        self.groups = [
            cache_kind(req.kind)(req, entries, self.n_pages, self.n_slots, self.blocks_per_seq, dtype, self.device,
                                 window_step_tokens)
            for req, entries in by_request.items()]
        self._where: Dict[int, Tuple[object, int]] = {}
        for g in self.groups:
            for j, e in enumerate(g.entries):
                self._where[e] = (g, j)
        for i, (req, src) in enumerate(zip(kv_requests, cache_from)):
            if src is not None and req is not None:
                if src not in self._where:
                    raise CacheError(f"schedule entry {i} reads the cache of entry {src}, which owns none")
                if self._where[src][0].request != req:
                    raise CacheError(f"schedule entry {i} reads the cache of entry {src}, whose layout differs")

        self.states: Dict[int, torch.Tensor] = {}
        for i, (sreq, src) in enumerate(zip(state_requests, cache_from)):
            if sreq is not None and src is None:
                self.states[i] = torch.zeros((self.n_slots,) + tuple(sreq.shape), dtype=sreq.dtype, device=self.device)

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        slot = self.slots.take()
        self.lengths[slot] = 0
        for st in self.states.values():
            st[slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is freed but is not held")
        for g in self.groups:
            g.release(slot)
        self.lengths[slot] = 0
        self.slots.give_back(slot)

    def reserve(self, slot: int, new_length: int) -> None:
        """Make room for the sequence in ``slot`` to hold ``new_length`` tokens; called before
        the step that brings the tokens beyond ``lengths[slot]``."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not held")
        if new_length > self.max_seq_len:
            raise CacheError(f"a sequence of {new_length} tokens exceeds the cache's limit of {self.max_seq_len}")
        if self.window_step_tokens is not None and new_length - self.lengths[slot] > self.window_step_tokens:
            raise CacheError(f"a step of {new_length - self.lengths[slot]} tokens exceeds the promised {self.window_step_tokens}")
        for g in self.groups:
            g.reserve(slot, self.lengths[slot], new_length)

    def flush_tables(self) -> None:
        """Bring the device's block tables up to date (copies on the current stream)."""
        for g in self.groups:
            g.flush()

    # ------------------------------------------------------------------ views
    def view(self, entry: int) -> CacheView:
        src = self.cache_from[entry]
        owner = entry if src is None else src
        k = v = table = None
        if owner in self._where:
            g, j = self._where[owner]
            k, v, table = g.view(j)
        return CacheView(k=k, v=v, block_table=table, state=self.states.get(owner), writable=src is None)

    # ------------------------------------------------------------------ accounting
    def held_tokens(self) -> int:
        """Tokens held by live sequences, each rounded up to whole pages."""
        return sum(pages_for(self.lengths[s], PAGE) * PAGE for s in range(self.n_slots) if self.slots.is_held(s))

    def pages_held(self) -> List[int]:
        return [g.held() for g in self.groups]

    def pool_sizes(self) -> List[int]:
        return [g.pool_size() for g in self.groups]

    def bytes(self) -> int:
        n = sum(g.bytes() for g in self.groups)
        return n + sum(s.numel() * s.element_size() for s in self.states.values())
