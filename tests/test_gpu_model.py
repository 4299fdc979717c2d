"""The engine against the plain implementation, in float32 and bfloat16: each request alone
and whole; with its last 32 tokens one by one; in batches of unequal lengths whose shorter
requests end earlier, one batch after another so that slots and pages are used again; long
decoding; the first tokens of a sequence; padding rows."""
from __future__ import annotations

import pytest
import torch

from helpers import assert_close, config_dict, plain_logits, random_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
CONFIGS = ["tiny1", "tiny2", "tiny3"]


@pytest.fixture(scope="module")
def engines(model_folders):
    """(config name, dtype) -> (engine, folder); models are loaded once per module."""
    from kuiperllama_b200.engine import Engine, load_model
    made = {}

    def get(name: str, dtype: str, max_tokens: int = 64 * 48):
        key = (name, dtype, max_tokens)
        if key not in made:
            folder = model_folders(name, seed={"tiny1": 0, "tiny2": 1, "tiny3": 2}[name])
            with torch.inference_mode():
                model = load_model(folder, dtype=dtype, device="cuda:0")
                made[key] = (Engine(model, model.new_cache(max_tokens=max_tokens)), folder)
        return made[key]

    return get


def _whole(engine, tokens):
    from kuiperllama_b200.engine import SequenceInput
    with torch.inference_mode():
        slot = engine.alloc_slot()
        out = engine.step([SequenceInput(slot, tokens, list(range(len(tokens))))])
        engine.free_slot(slot)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_each_request_alone_and_whole(engines, name, dtype):
    engine, folder = engines(name, dtype)
    vocab = config_dict(name)["vocab_size"]
    for i, n in enumerate([1, 7, 33, 64, 65, 100]):
        tokens = random_tokens(n, vocab, seed=100 + i)
        assert_close(_whole(engine, tokens), plain_logits(folder, tokens), dtype, f"{name} whole prompt of {n}")
    assert engine.cache.slots.held() == 0 and engine.cache.pages_held() == [0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_last_32_tokens_one_by_one(engines, name, dtype):
    from kuiperllama_b200.engine import SequenceInput
    engine, folder = engines(name, dtype)
    vocab = config_dict(name)["vocab_size"]
    for n in (33, 90, 127):
        tokens = random_tokens(n, vocab, seed=200 + n)
        ref = plain_logits(folder, tokens)
        head = n - 32
        with torch.inference_mode():
            slot = engine.alloc_slot()
            got = [engine.step([SequenceInput(slot, tokens[:head], list(range(head)))])]
            for t in range(head, n):
                got.append(engine.step([SequenceInput(slot, [tokens[t]], [0])]))
            engine.free_slot(slot)
        got = torch.cat(got, dim=0)
        # the first wrong place says what is special about it (a prompt's end, the first decoded token)
        assert_close(got[:head], ref[:head], dtype, f"{name} prefill part of {n}")
        assert_close(got[head:head + 1], ref[head:head + 1], dtype, f"{name} first decoded token of {n}")
        assert_close(got, ref, dtype, f"{name} last 32 one by one of {n}")


def _run_batch(engine, requests, prefill_lens):
    """requests: token lists; prefill_lens[i] tokens go in the first step, the rest one by one.
    Returns the logits of every position of every request."""
    from kuiperllama_b200.engine import SequenceInput
    with torch.inference_mode():
        slots = [engine.alloc_slot() for _ in requests]
        out = [[] for _ in requests]
        logits = engine.step([SequenceInput(s, r[:p], list(range(p))) for s, r, p in zip(slots, requests, prefill_lens)])
        o = 0
        for i, p in enumerate(prefill_lens):
            out[i].append(logits[o:o + p])
            o += p
        done = list(prefill_lens)
        live = [i for i in range(len(requests)) if done[i] < len(requests[i])]
        for i in range(len(requests)):
            if i not in live:
                engine.free_slot(slots[i])
        while live:
            logits = engine.step([SequenceInput(slots[i], [requests[i][done[i]]], [0]) for i in live])
            for j, i in enumerate(live):
                out[i].append(logits[j:j + 1])
                done[i] += 1
            still = []
            for i in live:
                if done[i] < len(requests[i]):
                    still.append(i)
                else:
                    engine.free_slot(slots[i])          # a shorter request ends earlier
            live = still
    return [torch.cat(o, dim=0) for o in out], slots


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_batches_of_unequal_lengths_reuse_slots(engines, name, dtype):
    engine, folder = engines(name, dtype)
    vocab = config_dict(name)["vocab_size"]
    # (total length, tokens given in the first step); batch after batch on the same slots
    batches = [[(13, 5), (40, 9), (70, 64), (21, 20)], [(66, 1), (9, 9), (100, 70)], [(120, 65), (64, 33)]]
    used = []
    for b, shape in enumerate(batches):
        requests = [random_tokens(n, vocab, seed=300 + 10 * b + i) for i, (n, _) in enumerate(shape)]
        got, slots = _run_batch(engine, requests, [p for _, p in shape])
        used.append(slots)
        for i, (r, g) in enumerate(zip(requests, got)):
            ref = plain_logits(folder, r)
            p = shape[i][1]
            assert_close(g[:p], ref[:p], dtype, f"{name} batch {b} request {i}: prompt part")
            assert_close(g, ref, dtype, f"{name} batch {b} request {i}: all positions")
        assert engine.cache.slots.held() == 0 and engine.cache.pages_held() == [0]
    assert set(used[1]) & set(used[0]), "the second batch did not reuse a slot of the first"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(engines, dtype):
    """A 150-token prompt and 400 tokens one by one across many pages (tiny3, context 2048)."""
    from kuiperllama_b200.engine import SequenceInput
    engine, folder = engines("tiny3", dtype)
    tokens = random_tokens(550, config_dict("tiny3")["vocab_size"], seed=400)
    ref = plain_logits(folder, tokens)
    with torch.inference_mode():
        slot = engine.alloc_slot()
        got = [engine.step([SequenceInput(slot, tokens[:150], [149])])]
        for t in range(150, 550):
            got.append(engine.step([SequenceInput(slot, [tokens[t]], [0])]))
        engine.free_slot(slot)
    assert_close(torch.cat(got, dim=0), ref[149:], dtype, "tiny3 long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_first_tokens_of_a_sequence(engines, name, dtype):
    """A sequence fed one token at a time from its very first token."""
    from kuiperllama_b200.engine import SequenceInput
    engine, folder = engines(name, dtype)
    tokens = random_tokens(6, config_dict(name)["vocab_size"], seed=500)
    ref = plain_logits(folder, tokens)
    with torch.inference_mode():
        slot = engine.alloc_slot()
        got = torch.cat([engine.step([SequenceInput(slot, [t], [0])]) for t in tokens], dim=0)
        engine.free_slot(slot)
    assert_close(got, ref, dtype, f"{name} first tokens one by one")


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_rows_change_nothing(engines, dtype):
    from kuiperllama_b200.engine import SequenceInput
    engine, folder = engines("tiny2", dtype)
    vocab = config_dict("tiny2")["vocab_size"]
    reqs = [random_tokens(n, vocab, seed=600 + n) for n in (10, 3)]
    outs = []
    for pad in (0, 5):
        with torch.inference_mode():
            slots = [engine.alloc_slot() for _ in reqs]
            a = engine.step([SequenceInput(s, r[:-1], list(range(len(r) - 1))) for s, r in zip(slots, reqs)], pad_rows=pad)
            b = engine.step([SequenceInput(s, [r[-1]], [0]) for s, r in zip(slots, reqs)], pad_rows=pad)
            for s in slots:
                engine.free_slot(s)
        outs.append(torch.cat([a, b], dim=0))
    assert torch.equal(outs[0], outs[1]), "padding rows changed a logit"
    ref = torch.cat([plain_logits(folder, r)[:-1] for r in reqs] + [plain_logits(folder, r)[-1:] for r in reqs], dim=0)
    assert_close(outs[1], ref, dtype, "tiny2 with padding rows")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_batch_of_more_than_64_sequences(engines, dtype):
    """70 sequences of unequal lengths: their prompts in one step (more than 64 rows, ragged),
    then decode steps of 70 rows, which take the kernels for many tokens instead of those for few."""
    engine, folder = engines("tiny1", dtype, max_tokens=64 * 80)
    vocab = config_dict("tiny1")["vocab_size"]
    reqs = [random_tokens(4 + (i * 7) % 9, vocab, seed=1200 + i) for i in range(70)]
    got, _ = _run_batch(engine, reqs, [len(r) - 3 for r in reqs])
    for i in (0, 1, 33, 64, 65, 69):
        assert_close(got[i], plain_logits(folder, reqs[i]), dtype, f"tiny1 {dtype}: sequence {i} of 70")


@pytest.mark.parametrize("name", ["tiny2", "tiny3"])
def test_the_option_that_folds_the_norms_into_the_products(model_folders, name):
    """bfloat16 decode steps of up to four sequences with ``stream_fusion``: the output and down
    projections add into the residual stream themselves, the products after them apply 1 / rms
    in their epilogue, and the two norm kernels of a layer are not launched.  Same logits as the
    plain implementation within the bfloat16 tolerance."""
    from kuiperllama_b200.csrc import ops
    from kuiperllama_b200.engine import Engine, SequenceInput, load_model
    folder = model_folders(name, seed=3)
    vocab = config_dict(name)["vocab_size"]
    reqs = [random_tokens(n, vocab, seed=900 + n) for n in (70, 41)]
    launches = {}
    for fusion in (False, True):
        with torch.inference_mode():
            model = load_model(folder, dtype="bfloat16", device="cuda:0")
            model.stream_fusion = fusion
            engine = Engine(model, model.new_cache(max_tokens=64 * 8))
            before = ops.launch_count
            got, _ = _run_batch(engine, reqs, [30, 30])
            launches[fusion] = ops.launch_count - before
        for g, r in zip(got, reqs):
            assert_close(g, plain_logits(folder, r), "bfloat16", f"{name}, stream fusion {fusion}")
    # every decode step saves at least one norm kernel per layer (which ones depends on the sizes:
    # a product whose operands the tensor-core kernel refuses asks for the dense rows)
    layers = config_dict(name)["num_hidden_layers"]
    assert launches[False] - launches[True] >= 40 * (layers - 1) > 0, launches


@pytest.mark.parametrize("dtype", DTYPES)
def test_logits_do_not_depend_on_the_cut_in_float32_order(engines, dtype):
    """Whole, split and batched runs of one request agree with each other far inside the
    tolerance against the oracle: the kernels sum in an order that depends only on the
    token's own position."""
    from kuiperllama_b200.engine import SequenceInput
    engine, folder = engines("tiny2", dtype)
    vocab = config_dict("tiny2")["vocab_size"]
    tokens = random_tokens(80, vocab, seed=700)
    other = random_tokens(45, vocab, seed=701)
    whole = _whole(engine, tokens)
    got, _ = _run_batch(engine, [other, tokens], [45, 50])
    if dtype == "float32":
        assert torch.equal(got[1], whole), "float32 logits changed with the cut or the batch"
    else:
        assert_close(got[1], whole.float().cpu(), "bfloat16", "bf16 cut vs whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny2", "tiny3"])
def test_decode_steps_replayed_from_cuda_graphs(model_folders, name, dtype):
    """The decode step captured in a CUDA graph per batch size: batches shrink as requests end,
    a later batch reuses slots and graphs, pages are crossed while replaying."""
    from kuiperllama_b200.engine import Engine, SequenceInput, load_model
    folder = model_folders(name, seed={"tiny2": 1, "tiny3": 2}[name])
    vocab = config_dict(name)["vocab_size"]
    with torch.inference_mode():
        model = load_model(folder, dtype=dtype, device="cuda:0")
        engine = Engine(model, model.new_cache(max_tokens=64 * 12), use_graphs=True)
        for batch in range(2):
            shape = [(100, 60), (70, 62), (90, 3)]                        # (total, given at first)
            reqs = [random_tokens(n, vocab, seed=800 + 10 * batch + i) for i, (n, _) in enumerate(shape)]
            slots = [engine.alloc_slot() for _ in reqs]
            engine.step([SequenceInput(s, r[:p], []) for s, r, (_, p) in zip(slots, reqs, shape)])
            done = [p for _, p in shape]
            live = [0, 1, 2]
            got = [[] for _ in reqs]
            while live:
                logits = engine.decode_step([slots[i] for i in live], [reqs[i][done[i]] for i in live]).clone()
                for j, i in enumerate(live):
                    got[i].append(logits[j])
                    done[i] += 1
                for i in [i for i in live if done[i] == len(reqs[i])]:
                    engine.free_slot(slots[i])
                live = [i for i in live if done[i] < len(reqs[i])]
            for i, r in enumerate(reqs):
                assert_close(torch.stack(got[i]), plain_logits(folder, r)[shape[i][1]:], dtype, f"{name} graphs batch {batch} request {i}")
        assert engine.graph_sizes() == [1, 2, 3]
        from kuiperllama_b200.csrc import ops
        ops.check_status(torch.device("cuda:0"))


def test_captured_steps_beyond_the_limit_are_dropped_and_captured_again(model_folders):
    """With room for two captured steps, batches of 3, 2 and 1 sequences (twice) keep dropping the
    graph used longest ago and capturing it anew; the logits stay those of the plain implementation."""
    from kuiperllama_b200.engine import Engine, SequenceInput, load_model
    folder = model_folders("tiny3", seed=2)
    vocab = config_dict("tiny3")["vocab_size"]
    with torch.inference_mode():
        model = load_model(folder, dtype="bfloat16", device="cuda:0")
        engine = Engine(model, model.new_cache(max_tokens=64 * 12), use_graphs=True)
        engine.MAX_GRAPHS = 2
        for batch in range(2):
            shape = [(40, 30), (37, 30), (34, 30)]
            reqs = [random_tokens(n, vocab, seed=900 + 10 * batch + i) for i, (n, _) in enumerate(shape)]
            slots = [engine.alloc_slot() for _ in reqs]
            engine.step([SequenceInput(s, r[:p], []) for s, r, (_, p) in zip(slots, reqs, shape)])
            done = [p for _, p in shape]
            live = [0, 1, 2]
            got = [[] for _ in reqs]
            while live:
                logits = engine.decode_step([slots[i] for i in live], [reqs[i][done[i]] for i in live]).clone()
                assert len(engine._graphs) <= 2
                for j, i in enumerate(live):
                    got[i].append(logits[j])
                    done[i] += 1
                for i in [i for i in live if done[i] == len(reqs[i])]:
                    engine.free_slot(slots[i])
                live = [i for i in live if done[i] < len(reqs[i])]
            assert engine.graph_sizes() == [1, 2]
            for i, r in enumerate(reqs):
                assert_close(torch.stack(got[i]), plain_logits(folder, r)[shape[i][1]:], "bfloat16", f"tiny3 two graphs kept, batch {batch} request {i}")
        engine.check_device_errors()


def test_a_float16_checkpoint_in_a_float32_run_keeps_its_values(tmp_path, model_folders):
    """A folder stored in float16 (as Llama-2 checkpoints are): the float32 run uses exactly those
    values, not values rounded to bfloat16 on the way; the bfloat16 run rounds them once."""
    import shutil
    from safetensors.torch import load_file, save_file
    from kuiperllama_b200.engine import Engine, load_model
    src = model_folders("tiny1", seed=0)
    g = torch.Generator().manual_seed(5)
    half = {k: (v.float() * (1 + 2.0 ** -10 * torch.randint(-3, 4, v.shape, generator=g))).half()
            for k, v in load_file(f"{src}/model.safetensors").items()}      # values bfloat16 cannot hold
    assert any(not torch.equal(v.bfloat16().half(), v) for v in half.values())
    shutil.copy(f"{src}/config.json", tmp_path / "config.json")
    save_file(half, str(tmp_path / "model.safetensors"))
    tokens = random_tokens(40, config_dict("tiny1")["vocab_size"], seed=1300)
    ref = plain_logits(str(tmp_path), tokens)                                # the oracle reads float16 as float32: exact
    for dtype in DTYPES:
        with torch.inference_mode():
            model = load_model(str(tmp_path), dtype=dtype, device="cuda:0")
            got = _whole(Engine(model, model.new_cache(max_tokens=64)), tokens)
        assert_close(got, ref, dtype, f"tiny1 float16 checkpoint, {dtype} run")
    rounded = {k: v.bfloat16().float() for k, v in half.items()}
    import plain_llama
    coarse = plain_llama.forward_logits(rounded, plain_llama.read_config(str(tmp_path)), tokens)
    assert float((coarse - ref).abs().max()) > 20 * 2e-5 * float(ref.abs().max())   # the rounding the float32 run must not make is visible


@pytest.mark.parametrize("dtype", DTYPES)
def test_llama31_8b_layer_sizes_one_layer(tmp_path_factory, dtype):
    """One layer with the widths of Llama-3.1-8B (hidden 4096, 32 heads, 8 kv heads, head size
    128, intermediate 14336, llama3 rope scaling) and a cut vocabulary: the tensor-core kernels
    at the shapes they serve, against the plain implementation, whole and one by one."""
    from helpers import write_folder, TINY
    from kuiperllama_b200.engine import Engine, SequenceInput, load_model
    TINY["wide"] = {
        "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 1,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 2000,
        "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "tie_word_embeddings": False, "hidden_act": "silu",
    }
    folder = str(tmp_path_factory.mktemp("wide"))
    write_folder(folder, "wide", seed=7)
    tokens = random_tokens(150, 2000, seed=900)
    ref = plain_logits(folder, tokens)
    with torch.inference_mode():
        model = load_model(folder, dtype=dtype, device="cuda:0")
        engine = Engine(model, model.new_cache(max_tokens=64 * 8), use_graphs=(dtype == "bfloat16"))
        slot = engine.alloc_slot()
        got = [engine.step([SequenceInput(slot, tokens[:140], list(range(140)))])]
        for t in tokens[140:]:
            got.append(engine.decode_step([slot], [t]).clone())
        engine.free_slot(slot)
    assert_close(torch.cat(got), ref, dtype, f"8B-width layer, {dtype}", layers=1, stream="wide")
    from kuiperllama_b200.csrc import ops
    ops.check_status(torch.device("cuda:0"))
