"""Shared by the tests: the tiny configurations, model folders, and the oracle's logits."""
from __future__ import annotations

import functools
import json
import math
import os
from typing import Dict, List, Sequence

import torch

import plain_llama

# Two tiny configurations of the Llama decoder that differ in every size and option, and a
# third with a head size that is not hidden/heads and a long context for decoding tests.
TINY: Dict[str, dict] = {
    "tiny1": {   # Llama-2 style: MHA, no rope scaling, untied
        "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "intermediate_size": 172,
        "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 4, "vocab_size": 256,
        "max_position_embeddings": 128, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
        "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
    },
    "tiny2": {   # Llama-3 style: GQA group 3, llama3 rope scaling, tied, two stop tokens
        "architectures": ["LlamaForCausalLM"], "hidden_size": 192, "intermediate_size": 512,
        "num_hidden_layers": 3, "num_attention_heads": 6, "num_key_value_heads": 2, "vocab_size": 384,
        "max_position_embeddings": 256, "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 64},
        "tie_word_embeddings": True, "hidden_act": "silu", "bos_token_id": 5, "eos_token_id": [7, 9],
    },
    "tiny3": {   # explicit head_dim (heads * head_dim != hidden), GQA group 4, odd vocabulary, long context
        "architectures": ["LlamaForCausalLM"], "hidden_size": 320, "intermediate_size": 328,
        "num_hidden_layers": 2, "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64,
        "vocab_size": 1003, "max_position_embeddings": 2048, "rms_norm_eps": 3e-6, "rope_theta": 250000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 512},
        "tie_word_embeddings": False, "hidden_act": "silu", "eos_token_id": 3,
    },
    "tiny4": {   # head size 128 with 8 kv heads (group 2): the tensor-core attention kernels' other head size
        "architectures": ["LlamaForCausalLM"], "hidden_size": 256, "intermediate_size": 320,
        "num_hidden_layers": 2, "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128,
        "vocab_size": 777, "max_position_embeddings": 1024, "rms_norm_eps": 2e-5, "rope_theta": 1000000.0,
        "rope_scaling": None, "tie_word_embeddings": True, "hidden_act": "silu", "eos_token_id": 4,
    },
}

SEEDS = {"tiny1": 0, "tiny2": 1, "tiny3": 2, "tiny4": 4}


def config_dict(name: str, **overrides) -> dict:
    d = json.loads(json.dumps(TINY[name]))
    d.update(overrides)
    return d


def write_folder(folder: str, name: str, seed: int, std: float = 0.02, **overrides) -> None:
    """A model folder of random weights through the package's random-weights mode.  ``std`` 0.02
    is the workloads' figure; with 0.08 the scores of the tiny models spread over several units, so
    that the softmax has sharp peaks and a wrong scale, mask, position or page shows in the logits."""
    from kuiperllama_b200.config import config_from_dict
    from kuiperllama_b200.engine import write_random_model_folder
    write_random_model_folder(folder, config_from_dict(config_dict(name, **overrides)), seed, std=std)


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


@functools.lru_cache(maxsize=64)
def _plain_cached(folder: str, tokens: tuple) -> torch.Tensor:
    c = plain_llama.read_config(folder)
    w = plain_llama.read_weights(folder)
    return plain_llama.forward_logits(w, c, list(tokens))


def plain_logits(folder: str, tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence from the plain implementation."""
    return _plain_cached(folder, tuple(int(t) for t in tokens))


# Tolerances.
#
# float32: the engine differs from the oracle only by the order of sums; 2e-5 of the largest logit
# (observed: at most 8e-6, at the Llama-3.1-8B widths with the whole vocabulary).
#
# bfloat16, an error model checked against measurements.  Every layer rounds about nine tensors to
# bfloat16 on the way (normalised rows twice, q/k/v, probabilities, attention output, the two
# projections' results, the activation; relative rounding error 2^-8 / sqrt(3) * 0.74 = 1.7e-3 rms
# each), and the feed-forward roughly doubles what reaches it.  Each layer so adds independent noise
# of about 1 % of the size of what it adds to the residual stream; the logits' error relative to the
# largest logit is that noise relative to the final stream (both maxima sit about five standard
# deviations out), so it grows as sqrt(layers).  Measured at the Llama-3.1-8B widths, bfloat16
# against float32 on the same weights, 1 / 2 / 4 / 8 / 16 / 32 layers: 0.93 / 1.28 / 1.61 / 2.51 /
# 2.97 / 5.17 % of the largest logit, i.e. 0.93 % * sqrt(layers) within a tenth.  In the tiny
# configurations (weights N(0, 0.02) at widths of 64 to 320) the stream is mostly the embedding,
# which bfloat16 holds exactly, and the same law has the factor 0.3 to 0.4 % (observed 0.43 / 0.62 /
# 0.58 / 0.57 % for tiny1 to tiny4 with 2 / 3 / 2 / 2 layers).  The tolerance is three times the law.
BF16_NOISE_PER_LAYER = {"narrow": 3.6e-3, "wide": 9.3e-3}


def tolerance(dtype: str, ref: torch.Tensor, layers: int = 3, stream: str = "narrow") -> float:
    scale = float(ref.abs().max())
    if dtype == "float32":
        return 2e-5 * scale + 1e-6
    return 3.0 * BF16_NOISE_PER_LAYER[stream] * math.sqrt(layers) * scale + 1e-6


# The largest error seen per dtype and test label, relative to the reference's largest magnitude;
# conftest.py prints it at the end of a run so that the tolerances can be set from it.
OBSERVED: Dict[tuple, float] = {}


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "", layers: int = 3,
                 stream: str = "narrow") -> None:
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - ref).abs()
    tol = tolerance(dtype, ref, layers, stream)
    key = (dtype, " ".join(what.split(" ")[:2]).rstrip(",:"))
    OBSERVED[key] = max(OBSERVED.get(key, 0.0), float(err.max()) / (float(ref.abs().max()) + 1e-30))
    if float(err.max()) > tol:
        idx = int(err.reshape(err.shape[0], -1).max(dim=1).values.argmax()) if err.dim() > 1 else int(err.argmax())
        raise AssertionError(f"{what}: max abs error {float(err.max()):.3e} > {tol:.3e} "
                             f"(first axis index of the worst row: {idx}, scale {float(ref.abs().max()):.3e})")
