"""The generation loop's decisions with a fake backend on the CPU: batches one after another,
stop tokens, sequences that end earlier, slots handed back and reused."""
import pytest

from kuiperllama_b200.cache import PAGE
from kuiperllama_b200.engine.generate import GenerationStats, next_batch, run_requests, tokens_held


class FakeBackend:
    """The next token of a sequence is (sum of its tokens + its length) mod 50."""

    def __init__(self, n_slots):
        self.free = list(range(n_slots))[::-1]
        self.held = {}
        self.log = []
        self.max_live = 0

    def alloc_slot(self):
        s = self.free.pop()
        self.held[s] = None
        self.max_live = max(self.max_live, len(self.held))
        return s

    def free_slot(self, slot):
        assert slot in self.held, "slot freed twice"
        del self.held[slot]
        self.free.append(slot)
        self.log.append(("free", slot))

    @staticmethod
    def _next(seq):
        return (sum(seq) + len(seq)) % 50

    def prefill(self, slots, prompts, request_ids):
        assert len(set(slots)) == len(slots)
        self.log.append(("prefill", tuple(request_ids), tuple(slots)))
        out = []
        for s, p in zip(slots, prompts):
            assert self.held[s] is None, "prefill into a slot that still holds a sequence"
            self.held[s] = list(p)
            out.append(self._next(self.held[s]))
        return out                                                   # a handle: here simply the list

    def decode(self, slots, previous, take, request_ids, steps):
        self.log.append(("decode", tuple(request_ids), tuple(steps)))
        out = []
        for s, j in zip(slots, take):
            assert s in self.held, "a step for a slot that was handed back"
            self.held[s].append(previous[j])
            out.append(self._next(self.held[s]))
        return out

    def read(self, handle):
        self.log.append(("read", len(handle)))
        return list(handle)

    def select(self, handle, keep):
        return [handle[j] for j in keep]


def expected(prompt, max_new, stop=()):
    seq, new = list(prompt), []
    for _ in range(max_new):
        t = FakeBackend._next(seq)
        if t in stop:
            return new, "stop"
        seq.append(t)
        new.append(t)
    return new, "length"


def test_batches_follow_one_another_and_every_slot_comes_back():
    prompts = [[i + 1] * (i % 7 + 1) for i in range(11)]
    be = FakeBackend(4)
    stats = GenerationStats()
    res = run_requests(be, prompts, max_new_tokens=6, max_batch=4, stats=stats)
    assert [r.tokens for r in res] == [expected(p, 6)[0] for p in prompts]
    assert all(r.finish_reason == "length" for r in res)
    assert stats.batches == 3 and be.max_live == 4 and not be.held
    prefills = [e for e in be.log if e[0] == "prefill"]
    assert [e[1] for e in prefills] == [(0, 1, 2, 3), (4, 5, 6, 7), (8, 9, 10)]
    assert set(prefills[1][2]) == set(prefills[0][2])              # the second batch reuses the slots
    assert stats.prefill_tokens == sum(len(p) for p in prompts)
    assert stats.decode_tokens == 11 * 5 and stats.decode_steps == 3 * 5   # no step runs for nothing without stop tokens


def test_stop_tokens_end_a_sequence_early_and_are_left_out():
    prompts = [[3], [10, 11], [7, 7, 7], [1, 2, 3, 4]]
    stop = {FakeBackend._next([10, 11]), expected([7, 7, 7], 3)[0][2]}
    be = FakeBackend(8)
    res = run_requests(be, prompts, max_new_tokens=9, stop_ids=stop)
    for p, r in zip(prompts, res):
        want, why = expected(p, 9, stop)
        assert r.tokens == want and r.finish_reason == why
    assert res[1].tokens == [] and res[1].finish_reason == "stop"  # stopped at its first token
    assert not be.held
    # A step is started before the tokens that feed it are read, so a sequence that meets a stop
    # token has run one more step for nothing; after that it is gone: batches only shrink.
    sizes = [len(e[1]) for e in be.log if e[0] == "decode"]
    assert sizes[0] == 4 and sizes[1] < 4 and sizes == sorted(sizes, reverse=True)
    order = [e[0] for e in be.log]
    assert order[:3] == ["prefill", "decode", "read"]                  # one step ahead of the host
    # the stopped sequence's slot comes back as soon as its token has been read
    first_free = next(i for i, e in enumerate(be.log) if e[0] == "free")
    second_decode = [i for i, e in enumerate(be.log) if e[0] == "decode"][1]
    assert first_free < second_decode
    with_stop = run_requests(FakeBackend(8), prompts, max_new_tokens=9, stop_ids=stop, include_stop=True)
    assert with_stop[1].tokens == [FakeBackend._next([10, 11])]


def test_steps_are_counted_per_request_for_the_sampler():
    be = FakeBackend(4)
    run_requests(be, [[1], [2]], max_new_tokens=4)
    assert [e[2] for e in be.log if e[0] == "decode"] == [(1, 1), (2, 2), (3, 3)]


def test_cache_limits_shape_the_batches():
    lens = [10, 100, 64, 65, 1]
    assert tokens_held(10, 20, 1000) == PAGE and tokens_held(64, 1, 1000) == 2 * PAGE and tokens_held(100, 500, 128) == 128
    assert next_batch([0, 1, 2, 3, 4], lens, 10, max_batch=8, token_budget=5 * PAGE, max_seq_len=1000) == [0, 1, 2]
    assert next_batch([3, 4], lens, 10, max_batch=1, token_budget=1 << 20, max_seq_len=1000) == [3]
    with pytest.raises(ValueError, match="does not fit"):
        next_batch([1], lens, 10, max_batch=4, token_budget=PAGE, max_seq_len=1000)
    be = FakeBackend(8)
    res = run_requests(be, [[1] * 60, [2] * 30], max_new_tokens=50, max_seq_len=64, token_budget=2 * PAGE)
    assert len(res[0].tokens) == 4 and res[0].finish_reason == "context"     # 60 + 4 fills the cache's limit
    assert len(res[1].tokens) == 34 and res[1].finish_reason == "context"
    with pytest.raises(ValueError, match="empty prompt"):
        run_requests(FakeBackend(1), [[]], 3)
    with pytest.raises(ValueError, match="no room"):
        run_requests(FakeBackend(1), [[1] * 64], 3, max_seq_len=64)
    assert run_requests(FakeBackend(1), [[1]], 0)[0].tokens == []


def test_slots_are_handed_back_when_the_backend_raises():
    """An exception inside a batch (here: the third decode step) leaves no slot held, so the same
    cache serves the next call."""
    class Failing(FakeBackend):
        def decode(self, slots, previous, take, request_ids, steps):
            if steps[0] == 3:
                raise RuntimeError("the device said no")
            return super().decode(slots, previous, take, request_ids, steps)

    be = Failing(4)
    with pytest.raises(RuntimeError, match="the device said no"):
        run_requests(be, [[1, 2, 3], [4], [5, 6]], max_new_tokens=8, max_batch=4)
    assert be.held == {} and sorted(be.free) == [0, 1, 2, 3]
    ok = FakeBackend(4)
    ok.free, ok.held = be.free, be.held
    assert [len(r.tokens) for r in run_requests(ok, [[1, 2, 3], [4]], max_new_tokens=5, max_batch=4)] == [5, 5]


def test_default_cache_size_fits_the_device_not_the_configuration():
    """Llama 3.1's config.json says 131072 positions; 64 such sequences would be a terabyte of keys
    and values.  The default is cut to a share of the memory that is free."""
    from kuiperllama_b200.api import DEFAULT_CACHE_FRACTION, default_cache_tokens
    per_token = 32 * 2 * 8 * 128 * 2                                  # Llama-3.1-8B in bfloat16: 128 KiB a token
    free = 160 * 10**9
    tokens = default_cache_tokens(per_token, max_batch=64, max_seq_len=131072, free_bytes=free)
    assert tokens % PAGE == 0 and tokens * per_token <= DEFAULT_CACHE_FRACTION * free
    assert tokens * per_token > 0.7 * free                             # and it does use what is there
    # a small model keeps the size it asked for; no room at all still gives one page
    assert default_cache_tokens(1024, max_batch=4, max_seq_len=100, free_bytes=free) == 4 * 2 * PAGE
    assert default_cache_tokens(per_token, 64, 131072, free_bytes=1000) == PAGE


def test_context_classes_and_the_pieces_planned_by_them(monkeypatch):
    """The class of a step's longest sequence (what a captured decode step is keyed by) and the number of
    pieces the decode attention cuts a sequence into for it: never more CTAs than one round holds where
    pieces are cut at all, never fewer pieces for a longer context, and one piece where the pairs of
    (sequence, kv head) fill the machine by themselves."""
    from kuiperllama_b200.csrc import ops
    from kuiperllama_b200.engine.step import context_class
    assert [context_class(n) for n in (0, 1, PAGE * 16, PAGE * 16 + 1, PAGE * 32, PAGE * 32 + 1, 131072)] == [0, 0, 0, 1, 1, 2, 7]
    monkeypatch.setattr(ops, "sm_count", lambda: 148)
    for head_dim, per_sm in ((128, 3), (64, 4)):
        for kv in (1, 4, 8, 32):
            for n_seqs in (1, 2, 3, 8, 16, 31, 32, 37, 64, 200):
                pieces = [ops.decode_attention_splits(n_seqs, kv, head_dim, c) for c in range(9)]
                assert pieces == sorted(pieces) and pieces[0] >= 1, (head_dim, kv, n_seqs, pieces)
                pairs = n_seqs * kv
                for c, s in enumerate(pieces):
                    if s > 2:
                        assert pairs * s <= per_sm * 148, (head_dim, kv, n_seqs, c, s)
                    if s == 2:
                        assert pairs * s <= 4 * 148
                if pairs > 2 * 148:
                    assert pieces[-1] == 1
    assert ops.decode_attention_splits(8, 8, 128, 0) == 6 and ops.decode_attention_splits(8, 8, 128, 5) == 6
    assert ops.decode_attention_splits(1, 8, 128, 0) == 16 and ops.decode_attention_splits(1, 8, 128, 5) == 55
    assert ops.decode_attention_splits(32, 8, 128, 2) == 1 and ops.decode_attention_splits(32, 8, 128, 3) == 2
