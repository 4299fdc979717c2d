"""Thirty random configurations of the architecture through the engine, in float32 and bfloat16,
against the plain implementation: head sizes 16 to 256 in steps of 16, one to eight kv heads with
groups of one to eight, widths and vocabularies that are no power of two (some with rows that are
not 16-byte aligned, which take the plain kernels), one to three layers, tied and untied, with and
without llama3 frequency scaling, three norm constants.  Each runs three ragged prompts in one step
(every place wanted) and then six decode steps from CUDA graphs.  A size the kernels do not take
must be refused with an error, never answered wrongly; none of these is refused.

The weights are N(0, 0.03): with 0.08 and widths of 400 and more the scores of these models spread
over tens of units, and bfloat16's rounding of one score then moves whole probabilities (the
float32 path still agrees to 2e-5 there; the bfloat16 error model of helpers.py does not hold)."""
from __future__ import annotations

import random

import pytest
import torch

from helpers import assert_close, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


def _configuration(rng: random.Random) -> dict:
    kv = rng.choice([1, 2, 3, 4, 8])
    scaling = rng.choice([None, {"rope_type": "llama3", "factor": rng.choice([2.0, 8.0, 32.0]), "low_freq_factor": 1.0,
                                 "high_freq_factor": rng.choice([2.0, 4.0]),
                                 "original_max_position_embeddings": rng.choice([32, 64, 512])}])
    return {"architectures": ["LlamaForCausalLM"],
            "hidden_size": rng.choice([8, 24, 40, 72, 100, 136, 172, 200, 264, 328]) * rng.choice([1, 2]),
            "intermediate_size": rng.choice([48, 88, 172, 200, 256, 344, 520]), "num_hidden_layers": rng.choice([1, 2, 3]),
            "num_attention_heads": kv * rng.choice([1, 2, 3, 4, 8]), "num_key_value_heads": kv,
            "head_dim": rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 256]),
            "vocab_size": rng.choice([97, 255, 300, 777, 1003, 2049]), "max_position_embeddings": 512,
            "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-6]), "rope_theta": rng.choice([10000.0, 500000.0]),
            "rope_scaling": scaling, "tie_word_embeddings": rng.choice([True, False]), "hidden_act": "silu"}


@pytest.mark.parametrize("index", range(30))
def test_a_random_configuration(tmp_path, index):
    from kuiperllama_b200.config import config_from_dict
    from kuiperllama_b200.engine import Engine, SequenceInput, load_model, write_random_model_folder
    rng = random.Random(7000 + index)
    cfg = _configuration(rng)
    what = (f"head {cfg['head_dim']}, {cfg['num_attention_heads']}/{cfg['num_key_value_heads']} heads, width {cfg['hidden_size']}, "
            f"inner {cfg['intermediate_size']}, vocabulary {cfg['vocab_size']}")
    folder = str(tmp_path)
    write_random_model_folder(folder, config_from_dict(cfg), index, std=0.03)
    steps, layers = 6, cfg["num_hidden_layers"]
    reqs = [random_tokens(rng.choice([1, 3, 17, 63, 64, 65, 130, 200]) + steps, cfg["vocab_size"], seed=100 * index + j) for j in range(3)]
    for dtype in ("float32", "bfloat16"):
        with torch.inference_mode():
            model = load_model(folder, dtype=dtype, device="cuda:0")
            engine = Engine(model, model.new_cache(max_tokens=64 * 16), use_graphs=True)
            slots = [engine.alloc_slot() for _ in reqs]
            first = engine.step([SequenceInput(s, r[:-steps], list(range(len(r) - steps))) for s, r in zip(slots, reqs)])
            rows = [engine.decode_step(slots, [r[len(r) - steps + k] for r in reqs]).clone() for k in range(steps)]
            engine.check_device_errors()
        at = 0
        for j, r in enumerate(reqs):
            ref = plain_logits(folder, r)
            n = len(r) - steps
            assert_close(first[at:at + n], ref[:n], dtype, f"random configuration ({what}): prompt {j}", layers=layers, stream="wide")
            at += n
            assert_close(torch.stack([rows[k][j] for k in range(steps)]), ref[n:], dtype,
                         f"random configuration ({what}): decode {j}", layers=layers, stream="wide")
