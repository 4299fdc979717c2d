"""Seeded random schedules against the plain implementation: requests join a running batch with a
whole prompt, a chunk of one or a single token, several sequences advance by unequal amounts in one
step, decode steps go through ``decode_step`` (CUDA graphs, several batch sizes and context
classes) or through ``step``, requests end and their slots are taken by later ones, and the wanted
places are a random subset of each step's tokens.  Every wanted row is compared; at the end no slot
and no page may be held."""
from __future__ import annotations

import random

import pytest
import torch

from helpers import SEEDS, assert_close, config_dict, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny3", "tiny4"])
def test_random_schedules(model_folders, name, dtype):
    from kuiperllama_b200.engine import Engine, SequenceInput, load_model
    folder = model_folders(name, seed=SEEDS[name], std=0.08, max_position_embeddings=2304)
    vocab = config_dict(name)["vocab_size"]
    with torch.inference_mode():
        model = load_model(folder, dtype=dtype, device="cuda:0")
        engine = Engine(model, model.new_cache(max_tokens=64 * 60, max_slots=6), use_graphs=True)
        for round_ in range(3):
            rng = random.Random(9000 + round_)
            live, finished, got, next_id = {}, [], {}, 0          # live: id -> [slot, tokens, done]
            for _ in range(rng.randrange(12, 36)):
                while len(live) < 6 and rng.random() < 0.35:
                    n = rng.choice([1, 2, 30, 64, 65, 100, 260, 700, 1100])
                    live[next_id] = [engine.alloc_slot(), random_tokens(n, vocab, seed=90000 + 100 * round_ + next_id), 0]
                    got[next_id] = []
                    next_id += 1
                if not live:
                    continue
                chosen = [i for i in live if rng.random() < 0.8] or [next(iter(live))]
                one_token_each = rng.random() < 0.5
                inputs, plan = [], []
                for i in chosen:
                    slot, tokens, done = live[i]
                    n = 1 if one_token_each else min(len(tokens) - done, rng.choice([1, 1, 5, 63, 64, 130, 300, 600]))
                    want = [0] if one_token_each else sorted(rng.sample(range(n), min(n, rng.choice([0, 1, 2, 5]))))
                    inputs.append(SequenceInput(slot, tokens[done:done + n], want))
                    plan.append((i, done, n, want))
                if one_token_each and rng.random() < 0.7:
                    logits = engine.decode_step([x.slot for x in inputs], [x.tokens[0] for x in inputs])
                else:
                    logits = engine.step(inputs)
                row = 0
                for i, done, n, want in plan:
                    for w in want:
                        got[i].append((done + w, logits[row].clone()))
                        row += 1
                    live[i][2] += n
                    if live[i][2] == len(live[i][1]):
                        engine.free_slot(live[i][0])
                        finished.append((i, live.pop(i)[1]))
            for i, (slot, tokens, done) in list(live.items()):
                engine.free_slot(slot)
                finished.append((i, tokens[:done]))
            engine.check_device_errors()
            assert engine.cache.slots.held() == 0 and engine.cache.pages_held() == [0]
            for i, tokens in finished:
                if got[i] and tokens:
                    ref = plain_logits(folder, tokens)
                    places = [p for p, _ in got[i]]
                    assert_close(torch.stack([r for _, r in got[i]]), ref[places], dtype,
                                 f"{name} random schedule {round_}, request {i} ({len(tokens)} tokens)", layers=2, stream="wide")
