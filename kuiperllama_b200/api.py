"""The Python entry point: ``load`` a model folder, ``generate`` from token ids.

ExiledOfCode/KuiperLLama has no Python binding; its two entry points are the C++ demo
(``llama_infer <checkpoint> <tokenizer>``, demo/main.cpp:50-75) and the ``generate`` method of
its PyTorch model (tools/model.py:315-343: ``generate(idx, max_new_tokens, temperature,
top_k)``).  The names and meanings of ``max_new_tokens``, ``temperature`` (0 picks the most
likely token) and ``top_k`` follow the latter; token ids go in and come out, as there.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

import torch

from .cache import PAGE, pages_for
from .engine.generate import EngineBackend, GenerationStats, RequestResult, run_requests
from .engine.loading import load_model, random_model
from .engine.model import DecoderModel
from .engine.step import Engine
from .sampling import Sampler, SamplingParams

# Share of the device memory that is free after the weights which a cache of default size may take.
DEFAULT_CACHE_FRACTION = 0.8


def default_cache_tokens(bytes_per_token: int, max_batch: int, max_seq_len: int, free_bytes: int,
                         fraction: float = DEFAULT_CACHE_FRACTION) -> int:
    """Tokens (a multiple of the page size) a cache holds when the caller names no size: room for
    ``max_batch`` sequences of ``max_seq_len``, but never more than ``fraction`` of the memory
    that is free, and at least one page.  A configuration's ``max_position_embeddings`` (131072
    for Llama 3.1) therefore never sizes the cache beyond what the device has."""
    want = max_batch * pages_for(max_seq_len, PAGE) * PAGE
    if bytes_per_token > 0:
        fits = int(free_bytes * fraction) // bytes_per_token // PAGE * PAGE
        want = min(want, fits)
    return max(PAGE, want)


class Inference:
    """A loaded model with its cache, step function and generation loop.

    ``max_tokens`` sizes the cache: the most tokens that live sequences hold at any time,
    each rounded up to whole pages of 64 (default: ``max_batch`` sequences of ``max_seq_len``,
    cut to what fits the free device memory).  ``max_batch`` bounds the sequences that run
    together and is the number of slots; ``max_seq_len`` bounds one sequence (default:
    max_position_embeddings).
    ``stream_fusion``: decode steps of up to 4 sequences fold the residual add and the norms
    into the products (about 3 % faster there; results differ in rounding from larger steps)."""

    def __init__(self, model: DecoderModel, max_tokens: Optional[int] = None, max_batch: int = 64,
                 max_seq_len: Optional[int] = None, use_graphs: bool = True, stream_fusion: bool = False):
        self.model = model
        model.stream_fusion = bool(stream_fusion) and model.runtime.dtype == torch.bfloat16
        self.max_seq_len = min(max_seq_len or model.spec.max_positions, model.spec.max_positions)
        self.max_batch = max_batch
        if max_tokens is None:
            free, _ = torch.cuda.mem_get_info(model.runtime.device)
            max_tokens = default_cache_tokens(model.cache_bytes_per_token(), max_batch, self.max_seq_len, free)
        self.cache = model.new_cache(max_tokens=max_tokens, max_seq_len=self.max_seq_len, max_slots=max_batch)
        self.max_seq_len = self.cache.max_seq_len
        self.engine = Engine(model, self.cache, use_graphs=use_graphs)
        self.last_stats: Optional[GenerationStats] = None
        self.last_results: Optional[List[RequestResult]] = None

    @property
    def stop_token_ids(self):
        return self.model.spec.stop_token_ids

    @torch.inference_mode()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, temperature: float = 0.0,
                 top_k: Optional[int] = None, seed: int = 0, stop_ids: Optional[Iterable[int]] = None,
                 include_stop: bool = False, return_logprobs: bool = False, return_logits: bool = False) -> List[List[int]]:
        """New token ids for every prompt (lists of token ids), in the order given.

        ``temperature`` 0 is greedy; otherwise softmax(logits / temperature) after an optional
        ``top_k`` cut, drawn with a generator keyed by (seed, index of the prompt, step).
        ``stop_ids`` default to the configuration's eos ids; a stop token ends its sequence
        and is left out unless ``include_stop``.

        With ``return_logprobs`` / ``return_logits`` the results in ``last_results`` also hold,
        for every new token, log softmax(logits)[token] of the model's own distribution
        (temperature 1, no cut) / the float32 logits row it was chosen from (host tensors).

        Before it returns, the device's report words are read: a kernel that gave up a bounded
        wait, or a token id outside the vocabulary that reached the device, raises here instead of
        passing for a result.  After any exception the slots of the batch under way are free again."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        if single:
            prompts = [prompts]
        sampler = Sampler(SamplingParams(temperature=float(temperature), top_k=top_k, seed=int(seed)))
        stats = GenerationStats()
        backend = EngineBackend(self.engine, sampler, logprobs=return_logprobs, logits=return_logits)
        try:
            results = run_requests(backend, [list(p) for p in prompts], int(max_new_tokens),
                                   stop_ids=self.stop_token_ids if stop_ids is None else stop_ids,
                                   include_stop=include_stop, max_batch=self.max_batch,
                                   token_budget=self.cache.n_pages * PAGE, max_seq_len=self.max_seq_len, stats=stats,
                                   want_details=return_logprobs or return_logits)
        except BaseException:
            try:                                          # clear the words: a later call must not be blamed for them
                self.engine.check_device_errors()
            except Exception:
                pass
            raise
        self.engine.check_device_errors()                 # one copy of two words; the loop's last read has synchronised
        self.last_stats, self.last_results = stats, results
        out = [r.tokens for r in results]
        return out[0] if single else out


# The name the entry class had when the Llama decoder was the only architecture in sight.
LlamaInfer = Inference


def load(path: Optional[str] = None, dtype: str = "bfloat16", device: str = "cuda:0", *, config=None,
         random_weights: bool = False, seed: int = 0, max_tokens: Optional[int] = None, max_batch: int = 64,
         max_seq_len: Optional[int] = None, use_graphs: bool = True, stream_fusion: bool = False) -> Inference:
    """Load the model folder ``path`` (config.json + model.safetensors).  With
    ``random_weights`` build a random model on the device instead, from ``config`` (a
    configuration object, a dict of config.json's keys, or the path of a config.json) or from
    the folder's config.json."""
    if random_weights:
        from .config import config_from_dict, config_from_file, config_from_folder
        if config is None:
            config = config_from_folder(path)
        elif isinstance(config, dict):
            config = config_from_dict(config)
        elif isinstance(config, str):
            config = config_from_file(config)
        model = random_model(config, seed, dtype=dtype, device=device)
    else:
        if path is None:
            raise ValueError("load() needs a model folder, or random_weights=True with a config")
        model = load_model(path, dtype=dtype, device=device)
    return Inference(model, max_tokens=max_tokens, max_batch=max_batch, max_seq_len=max_seq_len, use_graphs=use_graphs,
                     stream_fusion=stream_fusion)
