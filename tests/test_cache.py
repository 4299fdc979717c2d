"""The cache's bookkeeping on the CPU: no slot or page is lost, held twice or freed twice."""
import random

import pytest
import torch

from kuiperllama_b200.cache import PAGE, CacheError, FreeList, KVRequest, SequenceCache, StateRequest, pages_for


def test_free_list_hands_out_each_item_once():
    fl = FreeList(5, "slot")
    got = [fl.take() for _ in range(5)]
    assert sorted(got) == list(range(5)) and fl.available() == 0
    with pytest.raises(CacheError, match="no free slot"):
        fl.take()
    fl.give_back(3)
    with pytest.raises(CacheError, match="not held"):
        fl.give_back(3)                                            # freed twice
    with pytest.raises(CacheError, match="does not exist"):
        fl.give_back(9)
    assert fl.take() == 3                                          # the one just returned is reused first
    with pytest.raises(CacheError, match="wanted"):
        fl.take_many(2)


def _cache(max_tokens=PAGE * 10, max_seq_len=PAGE * 4, layers=3, state=False, cache_from=None):
    kv = [KVRequest(kv_heads=2, head_dim=16)] * layers
    st = [StateRequest((4,)) if state else None] * layers
    return SequenceCache(kv, st, cache_from or [None] * layers, max_tokens=max_tokens, max_seq_len=max_seq_len,
                         dtype=torch.float32, device="cpu")


def test_sizes_follow_max_tokens():
    c = _cache()
    assert c.n_pages == 10 and c.n_slots == 10 and c.blocks_per_seq == 4 and c.max_seq_len == PAGE * 4
    assert len(c.groups) == 1 and tuple(c.groups[0].k.shape) == (3, 10, 2, PAGE, 16)
    with pytest.raises(CacheError):
        _cache(max_tokens=PAGE - 1)
    assert _cache(max_tokens=PAGE * 2, max_seq_len=1000).max_seq_len == PAGE * 2


def test_pages_grow_with_the_sequence_and_come_back():
    c = _cache()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve(a, 1)
    c.reserve(b, PAGE + 1)
    assert c.pages_held() == [3]
    c.reserve(a, PAGE)                                            # still one page
    assert c.pages_held() == [3]
    c.reserve(a, PAGE + 1)
    assert c.pages_held() == [4]
    pa = list(c.groups[0].slot_pages[a])
    assert len(set(pa) | set(c.groups[0].slot_pages[b])) == 4       # no page held twice
    assert c.groups[0].table_host[a, :2].tolist() == pa
    with pytest.raises(CacheError, match="exceeds"):
        c.reserve(a, PAGE * 4 + 1)
    c.free_slot(a)
    assert c.pages_held() == [2] and c.slots.held() == 1
    with pytest.raises(CacheError, match="not held"):
        c.free_slot(a)                                             # freed twice
    with pytest.raises(CacheError, match="not held"):
        c.reserve(a, 5)
    a2 = c.alloc_slot()
    assert a2 == a                                                 # the slot is used again
    c.reserve(a2, 1)
    assert c.groups[0].slot_pages[a2][0] in pa                     # and so is one of its pages, stale contents and all


def test_pool_exhaustion_is_an_error_not_a_corruption():
    c = _cache(max_tokens=PAGE * 3, max_seq_len=PAGE * 3)
    s = [c.alloc_slot() for _ in range(3)]
    c.reserve(s[0], PAGE * 2)
    c.reserve(s[1], PAGE)
    with pytest.raises(CacheError, match="page"):
        c.reserve(s[2], 1)
    with pytest.raises(CacheError, match="no free slot"):
        c.alloc_slot()
    c.free_slot(s[0])
    c.reserve(s[2], PAGE * 2)
    assert c.pages_held() == [3]


def test_random_traffic_never_loses_or_doubles_anything():
    rng = random.Random(0)
    c = _cache(max_tokens=PAGE * 16, max_seq_len=PAGE * 5)
    live = {}
    for _ in range(3000):
        r = rng.random()
        if r < 0.3 and c.slots.available():
            live[c.alloc_slot()] = 0
        elif r < 0.8 and live:
            s = rng.choice(list(live))
            n = live[s] + rng.randint(1, 70)
            try:
                c.reserve(s, n)
                live[s] = n
                c.lengths[s] = n
            except CacheError:
                pass
        elif live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        g = c.groups[0]
        held = [p for s in live for p in g.pages_of(s)]
        assert len(held) == len(set(held)) == g.pages.held()
        assert all(len(g.slot_pages[s]) == pages_for(live[s], PAGE) for s in live)
        assert c.slots.held() == len(live)
        assert c.held_tokens() == sum(pages_for(n, PAGE) * PAGE for n in live.values())
    for s in list(live):
        c.free_slot(s)
    assert c.pages_held() == [0] and c.slots.held() == 0


def test_groups_with_different_needs_have_storage_of_their_own():
    kv = [KVRequest(2, 16), KVRequest(4, 32), KVRequest(2, 16), None, KVRequest(2, 16, window=8)]
    c = SequenceCache(kv, [None] * 5, [None] * 5, max_tokens=PAGE * 4, max_seq_len=PAGE * 2, dtype=torch.float32, device="cpu")
    assert len(c.groups) == 3
    shapes = sorted(tuple(g.k.shape) for g in c.groups)
    assert shapes == [(1, 4, 2, PAGE, 16), (1, 4, 4, PAGE, 32), (2, 4, 2, PAGE, 16)]
    s = c.alloc_slot()
    c.reserve(s, PAGE + 1)
    assert c.pages_held() == [2, 2, 2]
    assert c.view(0).k.data_ptr() != c.view(2).k.data_ptr() and c.view(0).block_table is c.view(2).block_table
    assert c.view(3).k is None and c.view(1).k.shape == (4, 4, PAGE, 32)
    c.free_slot(s)
    assert c.pages_held() == [0, 0, 0]


def test_reading_another_entrys_cache_and_state():
    c = _cache(layers=3, state=True, cache_from=[None, 0, None])
    assert c.view(1).k.data_ptr() == c.view(0).k.data_ptr() and not c.view(1).writable and c.view(0).writable
    assert tuple(c.groups[0].k.shape)[0] == 2                       # two owners only
    assert c.view(1).state.data_ptr() == c.view(0).state.data_ptr()
    s = c.alloc_slot()
    c.view(0).state[s] += 3.0
    c.free_slot(s)
    s2 = c.alloc_slot()
    assert s2 == s and float(c.view(0).state[s2].abs().sum()) == 0.0   # state is cleared when a slot is handed out
    with pytest.raises(CacheError):
        SequenceCache([None, KVRequest(2, 16)], [None, None], [None, 0], max_tokens=PAGE, max_seq_len=PAGE,
                      dtype=torch.float32, device="cpu")


def test_a_group_with_a_window_gives_back_the_pages_below_it():
    """Two groups: all keys, and a window of 100 keys.  While a sequence grows, the windowed
    group holds only the blocks from (length - window + 1) // PAGE on; no page is lost, held
    twice or given back twice, and everything returns when the slot is freed."""
    W = 100
    kv = [KVRequest(2, 16), KVRequest(2, 16, window=W)]
    c = SequenceCache(kv, [None] * 2, [None] * 2, max_tokens=PAGE * 32, max_seq_len=PAGE * 16, dtype=torch.float32, device="cpu")
    full, win = c.groups
    a, b = c.alloc_slot(), c.alloc_slot()
    lengths = {a: 0, b: 0}
    rng = random.Random(5)
    steps = [(a, 300), (b, 70)] + [(rng.choice([a, b]), 1) for _ in range(400)]
    for slot, n in steps:
        before = lengths[slot]
        if before + n > c.max_seq_len:
            continue
        c.reserve(slot, before + n)
        lengths[slot] = c.lengths[slot] = before + n
        for s, length in lengths.items():
            first_needed = max(0, (length - n if s == slot else length) - W + 1) // PAGE if length else 0
            # the windowed group keeps every block a query of the step just reserved can read ...
            assert all(p >= 0 for p in win.slot_pages[s][first_needed:])
            # ... and has given back everything below the window as it stood before that step
            assert win.first_block[s] <= first_needed
            assert len(full.pages_of(s)) == pages_for(length, PAGE)
        held = [p for s in lengths for p in win.pages_of(s)]
        assert len(held) == len(set(held)) == win.pages.held()
    assert win.first_block[a] > 0 and win.pages.held() < full.pages.held()
    # a sequence's windowed blocks never exceed the window plus two straddled pages
    assert all(len(win.pages_of(s)) <= pages_for(W, PAGE) + 2 for s in lengths)
    c.free_slot(a)
    c.free_slot(b)
    assert c.pages_held() == [0, 0]
    s2 = c.alloc_slot()
    c.reserve(s2, 10)
    assert win.first_block[s2] == 0 and len(win.pages_of(s2)) == 1


def test_a_windowed_group_can_have_a_smaller_pool():
    W = 100
    kv = [KVRequest(2, 16), KVRequest(2, 16, window=W)]
    c = SequenceCache(kv, [None] * 2, [None] * 2, max_tokens=PAGE * 64, max_seq_len=PAGE * 32, dtype=torch.float32, device="cpu",
                      max_slots=2, window_step_tokens=PAGE)
    assert c.pool_sizes() == [64, 2 * (pages_for(W + PAGE, PAGE) + 1)]
    s = c.alloc_slot()
    n = 0
    for step in [PAGE] * 20 + [1] * 100:
        c.reserve(s, n + step)
        n = c.lengths[s] = n + step
    assert c.pages_held()[0] == pages_for(n, PAGE) and c.pages_held()[1] <= pages_for(W + PAGE, PAGE) + 1
    with pytest.raises(CacheError):
        c.reserve(s, n + PAGE + 1)                          # more than the promised step
    c.free_slot(s)
    assert c.pages_held() == [0, 0]


def test_a_cache_kind_can_be_registered_from_outside():
    """Storage kinds are a registry like the parts: a kind defined here (a ring of one page per
    slot that keeps only the newest keys) is built for the executions that ask for it, beside the
    paged group of the others, and an unknown kind says which are known."""
    from kuiperllama_b200.cache import register_cache_kind

    @register_cache_kind("toy_last_page")
    class LastPage:
        def __init__(self, request, entries, n_pages, n_slots, blocks_per_seq, dtype, device, window_step_tokens=None):
            self.request, self.entries = request, entries
            self.k = torch.zeros((len(entries), n_slots, request.kv_heads, PAGE, request.head_dim), dtype=dtype, device=device)
            self.v = torch.zeros_like(self.k)
            self.table = torch.arange(n_slots, dtype=torch.int32, device=device).view(n_slots, 1)
            self.live = set()
            self.calls = []

        def reserve(self, slot, old_length, new_length):
            self.live.add(slot)
            self.calls.append((slot, old_length, new_length))

        def release(self, slot):
            self.live.discard(slot)

        def flush(self):
            pass

        def view(self, j):
            return self.k[j], self.v[j], self.table

        def held(self):
            return len(self.live)

        def pool_size(self):
            return self.k.shape[1]

        def bytes(self):
            return 2 * self.k.numel() * self.k.element_size()

    kv = [KVRequest(2, 16), KVRequest(2, 16, kind="toy_last_page"), KVRequest(2, 16)]
    c = SequenceCache(kv, [None] * 3, [None] * 3, max_tokens=PAGE * 6, max_seq_len=PAGE * 3, dtype=torch.float32, device="cpu",
                      max_slots=2)
    kinds = {type(g).__name__: g for g in c.groups}
    assert set(kinds) == {"PagedGroup", "LastPage"} and kinds["LastPage"].entries == [1]
    s = c.alloc_slot()
    c.reserve(s, 70)
    c.flush_tables()
    assert kinds["LastPage"].calls == [(s, 0, 70)] and sorted(c.pages_held()) == [1, 2]
    assert tuple(c.view(1).k.shape) == (2, 2, PAGE, 16) and tuple(c.view(0).k.shape) == (6, 2, PAGE, 16)
    c.free_slot(s)
    assert c.pages_held() == [0, 0]
    with pytest.raises(CacheError, match="toy_last_page"):          # the message lists the known kinds
        SequenceCache([KVRequest(2, 16, kind="nothing_like_it")], [None], [None], max_tokens=PAGE, max_seq_len=PAGE,
                      dtype=torch.float32, device="cpu")
