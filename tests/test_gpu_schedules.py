"""Schedules the step function allows beyond "prompts, then one token each", against the plain
implementation in float32 and bfloat16, for a head size of 64 (tiny3) and of 128 (tiny4):

* a prompt fed in several multi-token steps that cross page borders (a sequence that already
  holds tokens brings more than one: both tensor-core prefill kernels with ``seq_starts > 0``);
* a mixed step in which a fresh prompt joins sequences that are decoding;
* decode steps replayed from CUDA graphs at 8, 20, 33, 64, 96 and 130 sequences (the 16-, 32-, 64- and
  128-token tiles of the weights-as-rows products; decode attention with several pieces and with
  one piece per sequence; its light CTAs from 64 sequences of 8 kv heads on);
* the option that folds the norms into the products at 3 and 4 sequences.

The models here have weights N(0, 0.08), see ``SHARP``.
"""
from __future__ import annotations

import pytest
import torch

from helpers import SEEDS, assert_close, config_dict, plain_logits, random_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
CONFIGS = ["tiny3", "tiny4"]
# Weights N(0, 0.08) instead of N(0, 0.02): scores spread over several units, the softmax has sharp
# peaks, and a wrong scale, mask, position or page moves the logits far beyond the tolerance.
SHARP = 0.08
WIDE = dict(layers=2, stream="wide")


@pytest.fixture(scope="module")
def models(model_folders):
    from kuiperllama_b200.engine import load_model
    made = {}

    def get(name: str, dtype: str):
        if (name, dtype) not in made:
            folder = model_folders(name, seed=SEEDS[name], std=SHARP)
            with torch.inference_mode():
                made[(name, dtype)] = (load_model(folder, dtype=dtype, device="cuda:0"), folder)
        return made[(name, dtype)]

    return get


def _engine(model, max_tokens, use_graphs=False):
    from kuiperllama_b200.engine import Engine
    return Engine(model, model.new_cache(max_tokens=max_tokens), use_graphs=use_graphs)


@pytest.mark.parametrize("prefill_kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_a_prompt_in_several_multi_token_steps(models, name, dtype, prefill_kernel, monkeypatch):
    """300 tokens as steps of 70, 130, 9 and 91 tokens: every step but the first starts inside a
    page the sequence already holds part of, and ends in another."""
    from kuiperllama_b200.csrc import ops
    from kuiperllama_b200.engine import SequenceInput
    if dtype == "float32" and prefill_kernel == "mma":
        pytest.skip("the float32 path has one attention kernel")
    monkeypatch.setattr(ops, "PREFILL_KERNEL", prefill_kernel)
    model, folder = models(name, dtype)
    engine = _engine(model, 64 * 8)
    tokens = random_tokens(300, config_dict(name)["vocab_size"], seed=2100)
    ref = plain_logits(folder, tokens)
    got, start = [], 0
    with torch.inference_mode():
        slot = engine.alloc_slot()
        for n in (70, 130, 9, 91):
            got.append(engine.step([SequenceInput(slot, tokens[start:start + n], list(range(n)))]))
            assert_close(got[-1], ref[start:start + n], dtype, f"{name} {prefill_kernel}: the step of {n} tokens from {start}", **WIDE)
            start += n
        engine.free_slot(slot)
    engine.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_a_fresh_prompt_joins_decoding_sequences(models, name, dtype):
    """Two sequences are decoding; a step brings one token for each of them and a whole prompt of a
    third (and later of a fourth, a single token long); then all decode together."""
    from kuiperllama_b200.engine import SequenceInput
    model, folder = models(name, dtype)
    engine = _engine(model, 64 * 12)
    vocab = config_dict(name)["vocab_size"]
    reqs = [random_tokens(n, vocab, seed=2200 + n) for n in (90, 41, 77, 30)]
    ref = [plain_logits(folder, r) for r in reqs]
    done = [0, 0, 0, 0]
    got = [[] for _ in reqs]
    slots = {}

    def step(parts):                                    # parts: {request: number of tokens it brings}
        inputs = []
        for i, n in parts.items():
            if i not in slots:
                slots[i] = engine.alloc_slot()
            inputs.append(SequenceInput(slots[i], reqs[i][done[i]:done[i] + n], list(range(n))))
        logits = engine.step(inputs)
        o = 0
        for i, n in parts.items():
            got[i].append(logits[o:o + n])
            o += n
            done[i] += n

    with torch.inference_mode():
        step({0: 60, 1: 20})
        step({0: 1, 1: 1})
        step({0: 1, 1: 1, 2: 37})                       # the mixed step: a prompt of 37 joins
        step({0: 1, 1: 1, 2: 1})
        step({2: 1, 3: 1, 0: 1, 1: 1})                  # a prompt of one token joins, in another order
        while any(done[i] < len(reqs[i]) for i in range(4)):
            live = {i: 1 for i in range(4) if done[i] < len(reqs[i])}
            step(live)
            for i in list(slots):
                if done[i] == len(reqs[i]):
                    engine.free_slot(slots.pop(i))
    for i in range(4):
        assert_close(torch.cat(got[i]), ref[i], dtype, f"{name} request {i} of the mixed schedule", **WIDE)
    assert engine.cache.slots.held() == 0 and engine.cache.pages_held() == [0]
    engine.check_device_errors()


@pytest.mark.parametrize("batch", [8, 20, 33, 64, 80, 96, 130])
@pytest.mark.parametrize("name", CONFIGS)
def test_graph_decode_at_larger_batches(models, name, batch):
    """bfloat16 decode steps replayed from a CUDA graph at batch sizes that take the 16-, 32-, 64- and
    128-token tiles of the products (130: two tiles of tokens per weight tile) and every form of the
    decode attention; the same steps
    without a graph give the same bits, and both agree with the plain implementation."""
    from kuiperllama_b200.engine import SequenceInput
    model, folder = models(name, "bfloat16")
    vocab = config_dict(name)["vocab_size"]
    steps = 5
    reqs = [random_tokens(3 + (i * 11) % 70 + steps, vocab, seed=2300 + i) for i in range(batch)]
    outs = {}
    for use_graphs in (False, True):
        engine = _engine(model, 64 * 2 * batch, use_graphs=use_graphs)
        with torch.inference_mode():
            slots = [engine.alloc_slot() for _ in reqs]
            engine.step([SequenceInput(s, r[:-steps], []) for s, r in zip(slots, reqs)])
            rows = []
            for k in range(steps):
                rows.append(engine.decode_step(slots, [r[len(r) - steps + k] for r in reqs]).clone())
            for s in slots:
                engine.free_slot(s)
        outs[use_graphs] = torch.stack(rows, dim=1)          # [batch, steps, vocab]
        assert (engine.graph_sizes() == [batch]) == use_graphs
        engine.check_device_errors()
    assert torch.equal(outs[True], outs[False]), "a replayed graph gave other logits than the same kernels launched one by one"
    for i in sorted({0, 1, batch // 2, batch - 2, batch - 1}):
        assert_close(outs[True][i], plain_logits(folder, reqs[i])[-steps:], "bfloat16", f"{name} graph decode, sequence {i} of {batch}", **WIDE)


@pytest.mark.parametrize("name", CONFIGS)
def test_graph_decode_crosses_a_context_class(model_folders, name):
    """A sequence grows past 1,024 tokens while it decodes: the step is captured once more for the
    next class of context lengths (its decode attention is cut into other pieces there), and the
    logits on both sides of the border agree with the plain implementation and with the same
    steps launched kernel by kernel."""
    from kuiperllama_b200.engine import Engine, SequenceInput, load_model
    from kuiperllama_b200.engine.step import context_class
    assert [context_class(n) for n in (1, 1024, 1025, 2048, 2049, 4096, 4097)] == [0, 0, 1, 1, 2, 2, 3]
    folder = model_folders(name, seed=SEEDS[name], std=SHARP, max_position_embeddings=2304)
    vocab = config_dict(name)["vocab_size"]
    steps = 12
    reqs = [random_tokens(n + steps, vocab, seed=2500 + n) for n in (1018, 300)]
    outs = {}
    with torch.inference_mode():
        model = load_model(folder, dtype="bfloat16", device="cuda:0")
        for use_graphs in (False, True):
            engine = Engine(model, model.new_cache(max_tokens=64 * 24), use_graphs=use_graphs)
            slots = [engine.alloc_slot() for _ in reqs]
            for s, r in zip(slots, reqs):
                engine.step([SequenceInput(s, r[:-steps], [])])
            rows = [engine.decode_step(slots, [r[len(r) - steps + k] for r in reqs]).clone() for k in range(steps)]
            outs[use_graphs] = torch.stack(rows, dim=1)              # [2, steps, vocab]
            if use_graphs:
                assert sorted(engine._graphs) == [(2, 0), (2, 1)]
            engine.check_device_errors()
    assert torch.equal(outs[True], outs[False]), "replayed steps gave other logits than the same kernels launched one by one"
    for i, r in enumerate(reqs):
        ref = plain_logits(folder, r)[-steps:]
        for use_graphs in (False, True):
            assert_close(outs[use_graphs][i], ref, "bfloat16", f"{name} across the class border, graphs {use_graphs}, request {i}", **WIDE)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_small_steps_replayed_from_cuda_graphs(models, name, dtype):
    """Short prompts and chunks of prompts are captured too (rows padded to a multiple of 64).  Steps
    that share a key (sequences, padded rows, wanted places) but differ in lengths, start positions
    and slots replay one graph; their logits agree with the plain implementation and, in float32, are
    the bits of the same steps launched kernel by kernel without padding."""
    from kuiperllama_b200.engine import SequenceInput
    model, folder = models(name, dtype)
    vocab = config_dict(name)["vocab_size"]
    reqs = [random_tokens(n, vocab, seed=2600 + n) for n in (150, 97, 120, 33, 61)]
    ref = [plain_logits(folder, r) for r in reqs]
    # (request, tokens it brings) per step; wanted: the last place of every sequence of the step
    schedule = [[(0, 100)], [(1, 97)], [(0, 50), (2, 60)], [(2, 60), (3, 33)], [(4, 40)], [(4, 21)]]
    outs = {}
    for use_graphs in (False, True):
        engine = _engine(model, 64 * 16, use_graphs=use_graphs)
        done = [0] * len(reqs)
        slots = {}
        got = []
        with torch.inference_mode():
            for step in schedule:
                inputs = []
                for i, n in step:
                    if i not in slots:
                        slots[i] = engine.alloc_slot()
                    inputs.append(SequenceInput(slots[i], reqs[i][done[i]:done[i] + n], [n - 1]))
                logits = engine.step(inputs)
                for j, (i, n) in enumerate(step):
                    done[i] += n
                    got.append((i, done[i] - 1, logits[j].clone()))
        if use_graphs:
            # (1 sequence, 128 rows), (1, 64) used three times, (2, 128) used twice
            assert sorted(engine._step_graphs) == [(1, 64, 1), (1, 128, 1), (2, 128, 2)]
        engine.check_device_errors()
        outs[use_graphs] = got
    for (i, place, a), (_, _, b) in zip(outs[True], outs[False]):
        if dtype == "float32":       # (bfloat16: the padded rows change how the products cut their K range, so the last bits differ)
            assert torch.equal(a, b), f"request {i} place {place}: a captured small step gave other logits than the step launched kernel by kernel"
        assert_close(a[None], ref[i][place:place + 1], dtype, f"{name} small steps from graphs, request {i} place {place}", **WIDE)


@pytest.mark.parametrize("n_seqs", [3, 4])
@pytest.mark.parametrize("name", CONFIGS)
def test_stream_fusion_at_three_and_four_sequences(models, model_folders, name, n_seqs):
    from kuiperllama_b200.csrc import ops
    from kuiperllama_b200.engine import SequenceInput, load_model
    folder = model_folders(name, seed=SEEDS[name], std=SHARP)
    vocab = config_dict(name)["vocab_size"]
    steps = 12
    reqs = [random_tokens(20 + 13 * i + steps, vocab, seed=2400 + i) for i in range(n_seqs)]
    launches = {}
    for fusion in (False, True):
        with torch.inference_mode():
            model = load_model(folder, dtype="bfloat16", device="cuda:0")
            model.stream_fusion = fusion
            engine = _engine(model, 64 * 2 * n_seqs)
            slots = [engine.alloc_slot() for _ in reqs]
            engine.step([SequenceInput(s, r[:-steps], []) for s, r in zip(slots, reqs)])
            before = ops.launch_count
            rows = [engine.step([SequenceInput(s, [r[len(r) - steps + k]], [0]) for s, r in zip(slots, reqs)]) for k in range(steps)]
            launches[fusion] = ops.launch_count - before
        got = torch.stack(rows, dim=1)
        for i, r in enumerate(reqs):
            assert_close(got[i], plain_logits(folder, r)[-steps:], "bfloat16", f"{name} stream fusion {fusion}, {n_seqs} sequences", **WIDE)
        engine.check_device_errors()
    assert launches[True] < launches[False], launches
