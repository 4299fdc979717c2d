"""The Llama-3.1-8B shape itself (hidden 4096, 32 heads, 8 kv heads of 128, intermediate 14336,
the whole vocabulary of 128,256, llama3 rope scaling), under every way of cutting the work:

* two layers of it against the plain implementation on the CPU, in float32 and bfloat16;
* all 32 layers in bfloat16 against the engine's own float32 path on the same weights (the plain
  implementation cannot hold that model), with decode steps replayed from CUDA graphs at batch 8
  and one sequence taken past 3,000 tokens of context.

The cuts: a request alone and whole; its last 32 tokens one by one; a batch of unequal lengths
whose shorter requests end earlier, then a second batch on the slots and pages they gave back.
"""
from __future__ import annotations

import pytest
import torch

from helpers import BF16_NOISE_PER_LAYER, TINY, assert_close, plain_logits, random_tokens, write_folder

pytestmark = pytest.mark.gpu

LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "hidden_act": "silu",
}
VOCAB = LLAMA31_8B["vocab_size"]


# ------------------------------------------------------------------------------------------ two layers, CPU oracle

@pytest.fixture(scope="module")
def two_layer_folder(tmp_path_factory):
    TINY["llama31_8b_two_layers"] = dict(LLAMA31_8B, num_hidden_layers=2)
    folder = str(tmp_path_factory.mktemp("llama31-8b-two-layers"))
    write_folder(folder, "llama31_8b_two_layers", seed=11)
    return folder


def _drive(engine, requests, first, decode):
    """Run ``requests`` (token lists) as one batch: ``first[i]`` tokens in the first step, the rest
    one by one through ``decode`` (a function of (slots, tokens) -> logits); a request that has
    brought its last token gives its slot back at once.  Returns every request's logits at all
    its positions."""
    from kuiperllama_b200.engine import SequenceInput
    slots = [engine.alloc_slot() for _ in requests]
    out = [[] for _ in requests]
    logits = engine.step([SequenceInput(s, r[:p], list(range(p))) for s, r, p in zip(slots, requests, first)])
    o = 0
    for i, p in enumerate(first):
        out[i].append(logits[o:o + p].clone())
        o += p
    done = list(first)
    live = []
    for i, r in enumerate(requests):
        if done[i] < len(r):
            live.append(i)
        else:
            engine.free_slot(slots[i])
    while live:
        logits = decode([slots[i] for i in live], [requests[i][done[i]] for i in live])
        for j, i in enumerate(live):
            out[i].append(logits[j:j + 1].clone())
            done[i] += 1
        for i in [i for i in live if done[i] == len(requests[i])]:
            engine.free_slot(slots[i])
        live = [i for i in live if done[i] < len(requests[i])]
    return [torch.cat(o) for o in out], slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_layers_at_full_width_and_vocabulary_against_the_plain_implementation(two_layer_folder, dtype):
    from kuiperllama_b200.engine import Engine, SequenceInput, load_model
    folder = two_layer_folder
    reqs = {k: random_tokens(n, VOCAB, seed=3000 + n) for k, n in (("a", 150), ("b", 100), ("c", 45), ("d", 70), ("e", 20))}
    with torch.inference_mode():
        model = load_model(folder, dtype=dtype, device="cuda:0")
        engine = Engine(model, model.new_cache(max_tokens=64 * 10), use_graphs=(dtype == "bfloat16"))

        def decode(slots, tokens):
            return engine.decode_step(slots, tokens)

        # a request alone and whole
        (whole,), _ = _drive(engine, [reqs["a"]], [150], decode)
        assert_close(whole, plain_logits(folder, reqs["a"]), dtype, "8B-2-layers whole", layers=2, stream="wide")
        # its last 32 tokens one by one
        (split,), _ = _drive(engine, [reqs["a"]], [118], decode)
        assert_close(split[:118], plain_logits(folder, reqs["a"])[:118], dtype, "8B-2-layers prefill part", layers=2, stream="wide")
        assert_close(split[118:119], plain_logits(folder, reqs["a"])[118:119], dtype, "8B-2-layers first decoded token", layers=2, stream="wide")
        assert_close(split, plain_logits(folder, reqs["a"]), dtype, "8B-2-layers last 32 one by one", layers=2, stream="wide")
        if dtype == "float32":
            assert torch.equal(split, whole), "float32 logits changed with the cut"
        # a batch of unequal lengths whose shorter requests end earlier, then a batch on what they gave back
        got1, slots1 = _drive(engine, [reqs[k] for k in "abcd"], [100, 64, 45, 1], decode)
        got2, slots2 = _drive(engine, [reqs["e"], reqs["b"]], [10, 99], decode)
        for k, g in zip("abcd", got1):
            assert_close(g, plain_logits(folder, reqs[k]), dtype, f"8B-2-layers first batch, request {k}", layers=2, stream="wide")
        for k, g in zip("eb", got2):
            assert_close(g, plain_logits(folder, reqs[k]), dtype, f"8B-2-layers second batch, request {k}", layers=2, stream="wide")
        assert set(slots2) & set(slots1), "the second batch did not reuse a slot"
        if dtype == "float32":
            assert torch.equal(got1[0], whole)
        assert engine.cache.slots.held() == 0 and engine.cache.pages_held() == [0]
        engine.check_device_errors()


# ------------------------------------------------------------------------------------------ 32 layers, float32 path as oracle

@pytest.fixture(scope="module")
def full_models():
    """The 32-layer model twice on the device with the same (bfloat16-representable) weights: in
    float32 (32 GB, the oracle) and in bfloat16 (16 GB)."""
    from kuiperllama_b200.config import config_from_dict
    from kuiperllama_b200.engine import random_model
    free, _ = torch.cuda.mem_get_info()
    if free < 70e9:
        pytest.skip("the 32-layer float32 and bfloat16 models need about 60 GB of device memory")
    cfg = config_from_dict(LLAMA31_8B)
    with torch.inference_mode():
        oracle = random_model(cfg, seed=5, dtype="float32", device="cuda:0", stored="bfloat16")
        served = random_model(cfg, seed=5, dtype="bfloat16", device="cuda:0", stored="bfloat16")
    yield oracle, served
    del oracle, served
    torch.cuda.empty_cache()


def _oracle_rows(oracle_engine, tokens, want):
    """float32-path logits of one whole request at the places ``want``."""
    from kuiperllama_b200.engine import SequenceInput
    slot = oracle_engine.alloc_slot()
    out = oracle_engine.step([SequenceInput(slot, tokens, list(want))]).clone()
    oracle_engine.free_slot(slot)
    return out


def _assert_rows_noise(got, ref, what):
    """Row by row, the root-mean-square error over the 128,256 logits against the row's own
    root-mean-square: the noise of that position's final hidden state, which the error model puts
    at 0.93 % * sqrt(32) = 5.3 % (a statistic over so many logits that it barely scatters).  No row
    may show twice that: a position that read a wrong page or a wrong position's keys would."""
    got, ref = got.float().cpu(), ref.float().cpu()
    noise = (got - ref).pow(2).mean(dim=1).sqrt() / ref.pow(2).mean(dim=1).sqrt()
    worst = int(noise.argmax())
    assert float(noise.max()) < 2 * BF16_NOISE_PER_LAYER["wide"] * 32 ** 0.5, f"{what}: row {worst} has relative noise {float(noise.max()):.3f}"


def test_all_32_layers_in_bfloat16_against_the_float32_path(full_models):
    from kuiperllama_b200.engine import Engine, SequenceInput
    oracle, served = full_models
    with torch.inference_mode():
        oracle_engine = Engine(oracle, oracle.new_cache(max_tokens=64 * 50))
        engine = Engine(served, served.new_cache(max_tokens=64 * 120), use_graphs=True)

        # (1) a request alone and whole, and (2) with its last 32 tokens one by one past 3,000 tokens of context
        long = random_tokens(3050, VOCAB, seed=4000)
        places = list(range(0, 3018, 97)) + list(range(3018, 3050))
        ref = _oracle_rows(oracle_engine, long, places)
        slot = engine.alloc_slot()
        whole = engine.step([SequenceInput(slot, long, places)]).clone()
        engine.free_slot(slot)
        assert_close(whole, ref, "bfloat16", "8B whole request of 3,050 tokens", layers=32, stream="wide")
        _assert_rows_noise(whole, ref, "8B whole request of 3,050 tokens")
        slot = engine.alloc_slot()
        head = engine.step([SequenceInput(slot, long[:3018], [p for p in places if p < 3018])]).clone()
        tail = [engine.decode_step([slot], [t]).clone() for t in long[3018:]]
        engine.free_slot(slot)
        n_head = head.shape[0]
        assert_close(head, ref[:n_head], "bfloat16", "8B prefill part", layers=32, stream="wide")
        assert_close(tail[0], ref[n_head:n_head + 1], "bfloat16", "8B first decoded token at context 3,018", layers=32, stream="wide")
        assert_close(torch.cat(tail), ref[n_head:], "bfloat16", "8B last 32 one by one past 3,000 tokens", layers=32, stream="wide")
        _assert_rows_noise(torch.cat(tail), ref[n_head:], "8B last 32 one by one past 3,000 tokens")
        assert engine.graph_sizes() == [1]

        # (3) batches of 8 unequal requests through graphs; shorter ones end earlier; a second batch on their slots
        lengths1 = [(130, 100), (700, 690), (64, 40), (333, 320), (90, 89), (210, 180), (41, 33), (500, 470)]
        lengths2 = [(77, 50), (260, 255), (128, 100), (300, 290), (45, 20), (180, 150), (99, 98), (400, 380)]
        used = []
        for b, lengths in enumerate((lengths1, lengths2)):
            reqs = [random_tokens(n, VOCAB, seed=4100 + 50 * b + i) for i, (n, _) in enumerate(lengths)]
            got, slots = _drive(engine, reqs, [p for _, p in lengths], lambda s, t: engine.decode_step(s, t))
            used.append(slots)
            for i, (r, (n, p)) in enumerate(zip(reqs, lengths)):
                want = sorted(set(range(0, p, 53)) | set(range(p - 1, n)))       # some prompt places, every decoded one
                ref_rows = _oracle_rows(oracle_engine, r, want)
                assert_close(got[i][want], ref_rows, "bfloat16", f"8B batch {b} request {i} ({p} + {n - p} tokens)",
                             layers=32, stream="wide")
                _assert_rows_noise(got[i][want], ref_rows, f"8B batch {b} request {i}")
        assert set(used[0]) == set(used[1]), "the second batch did not run on the first one's slots"
        assert {1, 8} <= set(engine.graph_sizes())
        assert engine.cache.slots.held() == 0 and engine.cache.pages_held() == [0]
        engine.check_device_errors()
        oracle_engine.check_device_errors()
